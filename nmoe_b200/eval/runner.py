"""Snapshot evaluation runner (nmoe/eval/runner.py:237-409): load a model snapshot written by the training process, run
the multiple-choice and generation tasks of a task file within an example and a time budget, write ``summary.json``
next to the snapshot and the results into the metrics store.

  python -m nmoe_b200.eval.runner --snapshot DIR --run RUN --step N [--tasks core|NAME|chat:a|b] [--tasks-file F]
                                  [--max-examples 500] [--max-time-s 300] [--simulate --sim-acc-choices 0.6 ...]

Metric rows: ``eval/{task}/{acc,centered_acc,f1,n}``; the tags the reference's dashboards plot,
``eval/task/{task}/{acc,centered,n}`` and ``eval/CORE`` (mean centred accuracy of the multiple-choice tasks that ran).
``--simulate`` replaces the model by ``eval.simulate.SimulatedModel`` (target accuracies by hash): the whole path from
task file to dashboard can be checked before a long training run, without a GPU.
"""
from __future__ import annotations

import argparse
import json
import time
from pathlib import Path
from typing import Any, Dict, List, Optional

import torch


def select_tasks(tasks_file: str, which: str) -> Dict[str, Dict[str, Any]]:
  """Tasks of every kind for a selection: a group of the file (``core`` also takes ``core_gen``), one task name, or
  ``chat:name|name``.  Unknown names are left out."""
  from ..config import load_toml
  d = load_toml(tasks_file)    # expands ${NMOE_*:-default} placeholders
  tasks = d.get("tasks", d)
  groups = d.get("groups", {})
  if which.startswith("chat"):
    names = which.split(":", 1)[1].split("|") if ":" in which else list(groups.get("chat", []))
  elif which in groups:
    names = list(groups[which]) + list(groups.get(which + "_gen", []))
  elif which in tasks:
    names = [which]
  else:
    names = list(tasks) if which in ("", "all") else []
  return {n: tasks[n] for n in names if n in tasks and isinstance(tasks[n], dict)}


def _go_on(deadline: float) -> bool:
  """Whether there is budget for another task.  Rank 0 decides and tells the others: ranks that disagree about
  running a task would wait for each other in its collectives for ever."""
  import torch.distributed as dist
  ok = time.time() < deadline
  if dist.is_initialized() and dist.get_world_size() > 1:
    t = torch.tensor([int(ok)], device="cuda" if torch.cuda.is_available() and dist.get_backend() == "nccl" else "cpu")
    dist.broadcast(t, 0)
    ok = bool(t.item())
  return ok


def run_tasks(model, cfg, tasks: Dict[str, Dict[str, Any]], *, max_examples: int, max_time_s: float,
              rank: int = 0, world: int = 1) -> Dict[str, Dict[str, float]]:
  from ..data.transforms import get_tokenizer
  from .choices import eval_task
  from .run_gen import eval_gen_task
  enc = get_tokenizer(cfg.tokenizer)
  deadline = time.time() + max_time_s
  res: Dict[str, Dict[str, float]] = {}
  for name, t in tasks.items():
    if res and not _go_on(deadline):          # the first task always runs
      break
    if t.get("kind", "choices") == "choices":
      res[name] = eval_task(model, enc, t, rank=rank, world=world, max_examples=max_examples, pad_id=cfg.eos_token_id)
    else:
      res[name] = eval_gen_task(model, enc, name, t, rank=rank, world=world, max_examples=max_examples, eos_id=cfg.eos_token_id,
                                max_new=int(t.get("max_new", 64)))
  return res


def summarise(res: Dict[str, Dict[str, float]], requested: List[str], elapsed_s: float, suite: str) -> Dict[str, Any]:
  centred = [r["centered_acc"] for r in res.values() if "centered_acc" in r]
  return {"suite": suite, "CORE": sum(centred) / len(centred) if centred else 0.0,
          "tasks": [{"task": k, **v} for k, v in res.items()], "skipped": [n for n in requested if n not in res],
          "elapsed_s": round(elapsed_s, 3)}


def metric_rows(res: Dict[str, Dict[str, float]], core: float) -> List[tuple]:
  rows = [(f"eval/{t}/{k}", float(v)) for t, r in res.items() for k, v in r.items()]
  for t, r in res.items():
    rows += [(f"eval/task/{t}/acc", float(r["acc"])), (f"eval/task/{t}/n", float(r["n"]))]
    if "centered_acc" in r:
      rows.append((f"eval/task/{t}/centered", float(r["centered_acc"])))
  return rows + [("eval/CORE", float(core))]


def run_snapshot_eval(model, cfg, *, run_id: str, step: int, print_fn=print, tasks_file: Optional[str] = None,
                      max_examples: Optional[int] = None, which: Optional[str] = None, max_time_s: Optional[float] = None,
                      simulate=None) -> Dict:
  """Evaluate ``model`` (all ranks, in lockstep) or, with ``simulate`` (a ``SimConfig``), the stand-in; rank 0 records
  the results.  Returns the per-task results."""
  import torch.distributed as dist
  rank = dist.get_rank() if dist.is_initialized() else 0
  world = dist.get_world_size() if dist.is_initialized() else 1
  tasks = select_tasks(tasks_file or cfg.eval_tasks_file, which or cfg.eval_tasks)
  t0 = time.time()
  n_max = max_examples or cfg.eval_budget_max_examples
  if simulate is not None:
    from .simulate import simulate_suite
    res = simulate_suite(tasks, simulate, n_max)
  else:
    res = run_tasks(model, cfg, tasks, max_examples=n_max, max_time_s=cfg.eval_budget_max_time_s if max_time_s is None else max_time_s, rank=rank, world=world)
  summary = summarise(res, list(tasks), time.time() - t0, which or cfg.eval_tasks)
  if rank == 0:
    from .choices import format_results
    shown = {k: v for k, v in res.items() if "centered_acc" in v}
    print_fn(f"[eval] step {step}: CORE={summary['CORE']:.4f} {format_results(shown) if shown else ''} "
             + " ".join(f"{k}:acc={v['acc']:.3f}(n={int(v['n'])})" for k, v in res.items() if k not in shown)
             + (f" skipped={summary['skipped']}" if summary["skipped"] else "") + f" ({summary['elapsed_s']:.1f}s)")
    try:
      from ..metrics import MetricsWriter
      w = MetricsWriter(run_id, cfg.metrics_dir, 0)
      w.insert_many(step, metric_rows(res, summary["CORE"]))
      w.close()
    except OSError:
      pass
  run_snapshot_eval.last_summary = summary
  return res


def main(argv=None) -> None:
  ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
  ap.add_argument("--snapshot", required=True); ap.add_argument("--run", required=True); ap.add_argument("--step", type=int, required=True)
  ap.add_argument("--config", help="training configuration; default: config.json inside the snapshot")
  ap.add_argument("--tasks", help="group, task name or chat:a|b; default: the configuration's eval_tasks")
  ap.add_argument("--tasks-file"); ap.add_argument("--max-examples", type=int, default=500)
  ap.add_argument("--max-time-s", "--max-time", dest="max_time_s", type=int, default=300)
  ap.add_argument("--simulate", action="store_true", help="score a stand-in model with the accuracies below")
  ap.add_argument("--sim-acc-choices", type=float, default=0.6); ap.add_argument("--sim-acc-span", type=float, default=0.55)
  ap.add_argument("--sim-acc-unittest", type=float, default=0.5); ap.add_argument("--sim-acc-judge", type=float, default=0.6)
  ap.add_argument("--sim-seed", type=int, default=123)
  a = ap.parse_args(argv)
  from ..config import Config, from_toml
  snap = Path(a.snapshot)
  cfg = from_toml(a.config) if a.config else Config(**json.loads((snap / "config.json").read_text()))
  sim = model = None
  if a.simulate:
    from .simulate import SimConfig
    sim = SimConfig(a.sim_acc_choices, a.sim_acc_span, a.sim_acc_unittest, a.sim_acc_judge, a.sim_seed)
  else:
    from ..models.transformer import Transformer
    state = torch.load(snap / "model.pt", map_location="cpu", weights_only=False)
    dev = torch.device("cuda", 0) if torch.cuda.is_available() else torch.device("cpu")
    model = Transformer(cfg, dtype=torch.bfloat16 if dev.type == "cuda" else torch.float32, device=dev)
    model.load_state_dict(state["model"], strict=False)
  res = run_snapshot_eval(model, cfg, run_id=a.run, step=a.step, tasks_file=a.tasks_file, max_examples=a.max_examples,
                          which=a.tasks, max_time_s=a.max_time_s, simulate=sim)
  snap.mkdir(parents=True, exist_ok=True)
  (snap / "summary.json").write_text(json.dumps({"run": a.run, "step": a.step, "simulated": bool(a.simulate), "results": res,
                                                 **run_snapshot_eval.last_summary}, indent=1))


if __name__ == "__main__":
  main()
