"""Snapshot evaluation runner (nmoe/eval/runner.py:237-409): load a model snapshot written by the
training process, run the choice tasks within a time budget, write ``summary.json`` next to the
snapshot and the results into the metrics store under ``eval/*``."""
from __future__ import annotations

import argparse
import json
import time
from pathlib import Path
from typing import Dict, Optional

import torch


def run_snapshot_eval(model, cfg, *, run_id: str, step: int, print_fn=print, tasks_file: Optional[str] = None,
                      max_examples: Optional[int] = None) -> Dict:
  import torch.distributed as dist
  from .choices import format_results, run_eval
  rank = dist.get_rank() if dist.is_initialized() else 0
  world = dist.get_world_size() if dist.is_initialized() else 1
  t0 = time.time()
  res = run_eval(model, cfg, rank=rank, world=world, max_examples=max_examples or cfg.eval_budget_max_examples,
                 tasks_file=tasks_file)
  if rank == 0:
    print_fn(f"[eval] step {step}: {format_results(res)} ({time.time() - t0:.1f}s)")
    try:
      from ..metrics import MetricsWriter
      w = MetricsWriter(run_id, cfg.metrics_dir, 0)
      w.insert_many(step, [(f"eval/{t}/{k}", v) for t, r in res.items() for k, v in r.items()])
      w.close()
    except OSError:
      pass
  return res


def main(argv=None) -> None:
  ap = argparse.ArgumentParser()
  ap.add_argument("--snapshot", required=True); ap.add_argument("--run", required=True); ap.add_argument("--step", type=int, required=True)
  ap.add_argument("--config"); ap.add_argument("--tasks-file"); ap.add_argument("--max-examples", type=int, default=500)
  ap.add_argument("--max-time-s", type=int, default=300)
  a = ap.parse_args(argv)
  from ..config import Config, from_toml
  from ..models.transformer import Transformer
  snap = Path(a.snapshot)
  state = torch.load(snap / "model.pt", map_location="cpu", weights_only=False)
  cfg = from_toml(a.config) if a.config else Config(**json.loads((snap / "config.json").read_text()))
  dev = torch.device("cuda", 0) if torch.cuda.is_available() else torch.device("cpu")
  model = Transformer(cfg, dtype=torch.bfloat16 if dev.type == "cuda" else torch.float32, device=dev)
  model.load_state_dict(state["model"], strict=False)
  res = run_snapshot_eval(model, cfg, run_id=a.run, step=a.step, tasks_file=a.tasks_file, max_examples=a.max_examples)
  (snap / "summary.json").write_text(json.dumps({"run": a.run, "step": a.step, "results": res}, indent=1))


if __name__ == "__main__":
  main()
