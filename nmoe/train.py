"""``python -m nmoe.train <config.toml> [--key=value ...]`` -> ``nmoe_b200.train.main`` (same flags, same TOML), so launch
lines written for the reference (nmoe/train.py:1-12) keep working.  The directory deliberately has no ``__init__.py``:
as a namespace package it cannot shadow another installation of a package of the same name."""
from nmoe_b200.train import Trainer, main, train  # noqa: F401

if __name__ == "__main__":
  main()
