"""glog-style logging helpers: ``I0425 12:00:00.123 file.py:42] message`` (nmoe/log.py:7-86)."""
from __future__ import annotations

import logging
import os
import sys

_COLORS = {"D": "\033[36m", "I": "\033[32m", "W": "\033[33m", "E": "\033[31m", "C": "\033[35m"}


class GlogFormatter(logging.Formatter):
  def __init__(self, color: bool = False):
    super().__init__()
    self.color = color

  def format(self, record: logging.LogRecord) -> str:
    lvl = record.levelname[0]
    ts = self.formatTime(record, "%m%d %H:%M:%S")
    head = f"{lvl}{ts}.{int(record.msecs):03d} {record.filename}:{record.lineno}]"
    if self.color:
      head = f"{_COLORS.get(lvl, '')}{head}\033[0m"
    msg = record.getMessage()
    if record.exc_info:
      msg += "\n" + self.formatException(record.exc_info)
    return f"{head} {msg}"


def get_logger(name: str = "nmoe_b200") -> logging.Logger:
  lg = logging.getLogger(name)
  if not lg.handlers:
    h = logging.StreamHandler(sys.stderr)
    h.setFormatter(GlogFormatter(color=sys.stderr.isatty()))
    lg.addHandler(h)
    lg.setLevel(os.environ.get("NMOE_LOG_LEVEL", "INFO"))
    lg.propagate = False
  return lg


def rank() -> int:
  return int(os.environ.get("RANK", "0"))


def print0(*args, **kw) -> None:
  """print on rank 0 only."""
  if rank() == 0:
    print(*args, **kw, flush=True)


def check(cond: bool, msg: str) -> None:
  if not cond:
    raise RuntimeError(msg)
