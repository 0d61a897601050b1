"""Fixed-sequence-length reader over pre-tokenized ``.npy`` shards of uint32 token ids.

A ``Cursor`` names a position in the concatenation of the shard files; windows may cross file
boundaries and the stream wraps around at the end (``wrap_count`` increments), so a position is
fully described by three integers and resume is exact (nmoe/data/dataset.py:19-96).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Sequence, Tuple

import numpy as np


@dataclass
class Cursor:
  file_idx: int = 0
  pos_in_file: int = 0
  wrap_count: int = 0


class NumpyFSLDataset:
  def __init__(self, paths: Sequence[str]):
    if not paths:
      raise ValueError("NumpyFSLDataset needs at least one shard")
    self.paths: List[str] = list(paths)
    self._maps: List[np.ndarray | None] = [None] * len(self.paths)
    self._lens: List[int | None] = [None] * len(self.paths)

  def _open(self, i: int) -> np.ndarray:
    m = self._maps[i]
    if m is None:
      m = np.load(self.paths[i], mmap_mode="r")
      if m.ndim != 1:
        m = m.reshape(-1)
      self._maps[i] = m
      self._lens[i] = int(m.shape[0])
    return m

  def file_len(self, i: int) -> int:
    if self._lens[i] is None:
      self._open(i)
    return int(self._lens[i])

  def total_tokens(self) -> int:
    return sum(self.file_len(i) for i in range(len(self.paths)))

  def _normalize(self, c: Cursor) -> Cursor:
    fi, pos, wraps = c.file_idx, c.pos_in_file, c.wrap_count
    guard = 0
    while pos >= self.file_len(fi):
      pos -= self.file_len(fi)
      fi += 1
      if fi >= len(self.paths):
        fi = 0
        wraps += 1
      guard += 1
      if guard > 4 * len(self.paths) + 8:
        raise RuntimeError("shards are empty")
    return Cursor(fi, pos, wraps)

  def next_window(self, c: Cursor, n: int) -> Tuple[np.ndarray, Cursor]:
    """n consecutive tokens starting at ``c`` and the cursor advanced by n."""
    out = np.empty(n, dtype=np.uint32)
    c = self._normalize(c)
    filled = 0
    while filled < n:
      m = self._open(c.file_idx)
      take = min(n - filled, self.file_len(c.file_idx) - c.pos_in_file)
      out[filled:filled + take] = m[c.pos_in_file:c.pos_in_file + take]
      filled += take
      c = self._normalize(Cursor(c.file_idx, c.pos_in_file + take, c.wrap_count))
    return out, c

  def advance(self, c: Cursor, n: int) -> Cursor:
    """Cursor after skipping n tokens (no data is touched beyond file lengths)."""
    c = self._normalize(c)
    while n > 0:
      room = self.file_len(c.file_idx) - c.pos_in_file
      take = min(n, room)
      n -= take
      c = self._normalize(Cursor(c.file_idx, c.pos_in_file + take, c.wrap_count))
    return c

  def warmup(self, bytes_to_read: int = 64 << 20) -> None:
    """Touch the head of the first shard so the page cache is warm before step 0."""
    m = self._open(0)
    k = min(int(m.shape[0]), bytes_to_read // 4)
    if k:
      _ = int(np.asarray(m[:k]).sum(dtype=np.uint64))
