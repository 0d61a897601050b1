"""Entry-point alias: ``python -m nmoe.train cfg.toml`` and ``torchrun ... -m nmoe.train cfg.toml`` start the
trainer of the ``nmoe_b200`` package, so launch lines written for the reference (nmoe/train.py:1-12) keep working.
Everything else lives in ``nmoe_b200``; attribute access on this package is forwarded there."""
import importlib as _importlib

_impl = _importlib.import_module("nmoe_b200")


def __getattr__(name):
  try:
    return getattr(_impl, name)
  except AttributeError:
    return _importlib.import_module(f"nmoe_b200.{name}")
