"""``python -m nmoe.eval.choices <config.toml> ...`` -> ``nmoe_b200.eval.choices.main`` (nmoe/eval/choices.py:345-392)."""
from nmoe_b200.eval.choices import main, run_eval  # noqa: F401

if __name__ == "__main__":
  main()
