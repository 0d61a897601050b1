"""``python -m nmoe.train <config.toml> [--key=value ...]`` -> ``nmoe_b200.train.main`` (same flags, same TOML)."""
from nmoe_b200.train import Trainer, main, train  # noqa: F401

if __name__ == "__main__":
  main()
