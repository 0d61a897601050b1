"""``python -m nmoe.eval.runner --snapshot ...`` -> ``nmoe_b200.eval.runner.main`` (nmoe/eval/runner.py:237-409)."""
from nmoe_b200.eval.runner import main, run_snapshot_eval  # noqa: F401

if __name__ == "__main__":
  main()
