"""``python -m nmoe.eval.run_gen <config.toml> ...`` -> ``nmoe_b200.eval.run_gen.main`` (nmoe/eval/run_gen.py:198-339)."""
from nmoe_b200.eval.run_gen import main  # noqa: F401

if __name__ == "__main__":
  main()
