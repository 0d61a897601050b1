"""Scheduling of out-of-band evaluations during training (nmoe/eval/hooks.py:21-113).

``eval_mode``:
  inline        run the snapshot runner in this process right away (all ranks, lockstep)
  reserved_gpu  rank 0 saves a model snapshot and starts ``python -m nmoe_b200.eval.runner`` as a
                subprocess pinned to ``eval_reserved_gpu_id``
  k8s_job       rank 0 writes a ticket file ``{metrics_dir}/eval_tickets/{run}_{step}.json`` that an
                external controller turns into a job
"""
from __future__ import annotations

import json
import os
import subprocess
import sys
import time
from pathlib import Path

import torch


def save_eval_snapshot(model, cfg, run_id: str, step: int) -> Path:
  d = Path(cfg.checkpoint_dir) / "eval_snapshots" / f"{run_id}_step{step:07d}"
  d.mkdir(parents=True, exist_ok=True)
  torch.save({"step": step, "model": {k: v.detach().cpu() for k, v in model.state_dict().items()}}, d / "model.pt")
  # the runner rebuilds the model from the configuration it was trained with
  import dataclasses
  (d / "config.json").write_text(json.dumps({k: v for k, v in dataclasses.asdict(cfg).items() if not k.startswith("_")}, default=str))
  return d


def maybe_schedule_eval(step: int, cfg, model, run_id: str, print_fn=print):
  if not cfg.eval_enabled or cfg.eval_every <= 0 or step % cfg.eval_every != 0:
    return None
  rank = int(os.environ.get("RANK", "0"))
  if cfg.eval_mode == "inline":
    from .runner import run_snapshot_eval
    return run_snapshot_eval(model, cfg, run_id=run_id, step=step, print_fn=print_fn)
  if rank != 0:
    return None
  snap = save_eval_snapshot(model, cfg, run_id, step)
  if cfg.eval_mode == "reserved_gpu":
    env = dict(os.environ, CUDA_VISIBLE_DEVICES=str(cfg.eval_reserved_gpu_id), WORLD_SIZE="1", RANK="0", LOCAL_RANK="0")
    cmd = [sys.executable, "-m", "nmoe_b200.eval.runner", "--snapshot", str(snap), "--run", run_id, "--step", str(step),
           "--tasks-file", cfg.eval_tasks_file, "--tasks", cfg.eval_tasks, "--max-examples", str(cfg.eval_budget_max_examples),
           "--max-time-s", str(cfg.eval_budget_max_time_s)]
    p = subprocess.Popen(cmd, env=env, stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL)
    print_fn(f"[eval] step {step}: runner pid {p.pid} on GPU {cfg.eval_reserved_gpu_id}")
    return p
  if cfg.eval_mode == "k8s_job":
    t = Path(cfg.metrics_dir) / "eval_tickets"
    t.mkdir(parents=True, exist_ok=True)
    ticket = t / f"{run_id}_{step:07d}.json"
    ticket.write_text(json.dumps({"run": run_id, "step": step, "snapshot": str(snap), "tasks": cfg.eval_tasks,
                                  "tasks_file": cfg.eval_tasks_file, "created": time.time()}))
    print_fn(f"[eval] step {step}: ticket {ticket}")
    return ticket
  raise ValueError(f"unknown eval_mode {cfg.eval_mode!r}")
