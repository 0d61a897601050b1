"""Training entry point: ``python -m nmoe_b200.train <config.toml> [--key=value ...]`` or
``torchrun ... -m nmoe_b200.train <config.toml>``.

One path: forward -> masked CE -> backward -> optimizer step -> log -> eval -> checkpoint
(nmoe/train.py:36-184).  ``Trainer`` is the public step API; ``train(cfg)`` is the full loop
with data loading, metrics, experiment tracking and checkpoint/resume.
"""
from __future__ import annotations

import os
import sys
import time
from contextlib import nullcontext
from typing import Optional, Tuple

os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")

import torch
import torch.distributed as dist

from . import runtime
from .config import Config, fingerprint, from_toml
from .log import print0
from .models.transformer import Transformer
from .opt import Optimizer
from .utils.profiling import StepProfiler, scope


class Trainer:
  """Owns the model and optimizer of one rank and advances them one step at a time.

  ``step(inputs, targets)`` takes host (ideally pinned) or device int64 tensors of shape
  [micro_batch, seq_len], copies them to the device if needed, runs forward/backward/update and
  returns the loss as a device scalar (call ``.item()`` to read it on the host).
  """

  def __init__(self, cfg: Config, *, rank: int = 0, world: int = 1, device: Optional[torch.device] = None,
               fuse_expert_opt: Optional[bool] = None, init: bool = True):
    self.cfg, self.rank, self.world = cfg, rank, world
    self.device = device or torch.device("cpu")
    on_cuda = self.device.type == "cuda"
    dtype = torch.bfloat16 if on_cuda else torch.float32
    self.model = Transformer(cfg, dtype=dtype, device=self.device)
    if init:
      self.model.init_weights()
    self.model.train()
    if fuse_expert_opt is None:
      fuse_expert_opt = on_cuda and os.environ.get("NMOE_EXPERT_OPT_IN_BACKWARD", "1") == "1"
    self.opt = Optimizer(self.model, cfg, fuse_expert_in_backward=fuse_expert_opt)
    self.step_num = 0
    self.tokens_seen = 0
    self.gradnorm_sq = torch.zeros(1, dtype=torch.float32, device=self.device)
    self.track_gradnorm = False
    self.lr = 0.0
    self.nvtx = os.environ.get("NMOE_NVTX", "0") in ("1", "true", "True") and on_cuda
    # The host may queue at most one step ahead of the device.  Memory that a step hands to a side stream (expert
    # gradients to the optimizer stream, activations to the shared-expert stream) only returns to the allocator when that
    # stream has passed it; a host running two steps ahead asks for all of it twice, which at ~150 of 180 GB ends in
    # cudaMalloc retries inside the timed steps (measured: 450 ms per step instead of 395).  Waiting for the END of the
    # previous step costs nothing: queueing a step takes the host a quarter of the time the device needs to run it.
    self._step_end = [torch.cuda.Event(), torch.cuda.Event()] if on_cuda else None

  def _range(self, tag: str):
    return torch.cuda.nvtx.range(tag) if self.nvtx else nullcontext()

  def step(self, inputs: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
    if inputs.device != self.device:
      inputs = inputs.to(self.device, non_blocking=True)
      targets = targets.to(self.device, non_blocking=True)
    if self._step_end is not None and self.step_num > 0:
      self._step_end[(self.step_num - 1) & 1].synchronize()
    gn = None
    if self.track_gradnorm:
      self.gradnorm_sq.zero_()
      gn = self.gradnorm_sq
    self.opt.dense.gradnorm_sq = gn
    self.lr = self.opt.begin_step(self.step_num, self.tokens_seen, gn)
    with self._range("train/fwd_total"):
      loss = self.model.loss(inputs, targets)
    with self._range("train/bwd_total"), scope("backward"):
      loss.backward()
    with self._range("train/opt_step"), scope("optimizer"):
      self.opt.step()
    if self._step_end is not None:
      self._step_end[self.step_num & 1].record()
    self.step_num += 1
    self.tokens_seen += self.cfg.batch_size * self.cfg.seq_len
    return loss.detach()

  def grad_norm(self) -> torch.Tensor:
    """sqrt of the squared-gradient sum of the last step (all-reduced); needs track_gradnorm."""
    g = self.gradnorm_sq.clone()
    if dist.is_initialized() and self.world > 1:
      dist.all_reduce(g)
    return g.sqrt()


def train(cfg: Config) -> dict:
  from .checkpoint import Checkpointer, load_checkpoint, save_checkpoint
  from .data.loader import build_loader
  from .experiments import ExperimentTracker
  from .metrics import MetricsSession, log_training_step
  from .ops import tc_gemm

  rank, world, device = runtime.init(cfg.seed)
  cfg.validate(world)
  tracker = None
  run_id = os.environ.get("NMOE_RUN", "")
  if rank == 0:
    tracker = ExperimentTracker(cfg)
    run_id = tracker.start_run(run_id=run_id or None)
  checkpointer = Checkpointer(cfg.checkpoint_dir, keep_last=cfg.checkpoint_keep_last_n, async_io=True)
  loader, plan = build_loader(cfg, rank, world)
  trainer = Trainer(cfg, rank=rank, world=world, device=device)
  metrics = MetricsSession(run_id or f"run_{int(time.time())}", cfg.metrics_dir, rank, world, trainer.model, cfg)
  from .metrics import param_summary
  print0(f"[nmoe] {cfg.preset or 'model'} {param_summary(trainer.model, cfg, world)} on {world} rank(s), run {run_id}")
  start_step, tokens_seen = load_checkpoint(checkpointer, trainer, loader, plan, cfg, rank, print0)
  trainer.step_num, trainer.tokens_seen = start_step, tokens_seen
  fp = fingerprint(cfg)
  last_loss = None
  watch = tc_gemm.StatusWatch(device) if (device.type == "cuda" and world > 1) else None
  from .parallel.health import maybe_health
  health = maybe_health(rank, world, stall_s=float(os.environ.get("NMOE_PEER_STALL_S", "600")))
  if device.type == "cuda":
    tc_gemm.check_status_collective(device, world)      # nothing latched by set-up before the first step
  from .utils.stop import StopRequest
  stopper = StopRequest(world if dist.is_initialized() else 1)
  steps_done = cfg.steps
  profiler = StepProfiler(cfg.profiling_enabled, os.path.join(cfg.profiling_output_dir, run_id or "run"), rank,
                          steps=cfg.profiling_steps, skip=cfg.profiling_skip, print_fn=print)
  try:
    for step_num in range(start_step, cfg.steps):
      if health is not None:
        health.check()            # a peer that died or stalled is reported here, before this step's kernels wait on it
      t0 = time.perf_counter()
      inputs, targets = loader.next()
      loader_wait_ms = (time.perf_counter() - t0) * 1000.0
      s = step_num + 1
      trainer.track_gradnorm = (s % cfg.log_every == 0) or s == 1
      with metrics.timer("time_ms/step"):
        loss = trainer.step(inputs, targets)
      last_loss = loss
      profiler.step()
      log_training_step(metrics, s, trainer, loss, loader_wait_ms, print0)
      if health is not None:
        health.beat(s)
      if watch is not None:
        # multi-rank: peers depend on this rank's flags and buffers, so look at the record every step (copied
        # behind the step's kernels, examined when it has arrived: no host wait)
        watch.poll()
        watch.enqueue()
      if device.type == "cuda" and s % cfg.log_every == 0:
        tc_gemm.check_status(device)
      if cfg.eval_every > 0 and s % cfg.eval_every == 0:
        try:
          from .eval.choices import format_results, run_eval
          res = run_eval(trainer.model, cfg, rank=rank, world=world, max_examples=cfg.eval_budget_max_examples)
          print0(f"[eval] step={s} {format_results(res)}")
          metrics.insert_many(s, [(f"eval_choices/{t}/{k}", float(v)) for t, r in res.items() for k, v in r.items()
                                  if k in ("acc", "centered_acc", "n")])
        except Exception as e:  # evaluation must never take the run down
          print0(f"[eval] failed: {e}")
      try:
        from .eval.hooks import maybe_schedule_eval
        maybe_schedule_eval(s, cfg, trainer.model, run_id, print0)
      except Exception as e:
        print0(f"[eval] scheduling failed: {e}")
      stopping = stopper.should_stop(s)
      save_checkpoint(checkpointer, s, trainer, loader, plan, cfg, rank, fp, print0, force=stopping)
      if stopping:
        # a stop was asked for (SIGTERM from a scheduler, SIGUSR1 by hand): every rank is at this same step
        steps_done = s
        print0(f"[nmoe] stop requested ({stopper.reason or 'by another rank'}): checkpoint written at step {s}, leaving")
        break
    stopped = steps_done < cfg.steps
    if not stopped:
      print0(f"[nmoe] Training complete. {trainer.tokens_seen:,} tokens.")
    results = {"final_loss": float(last_loss.item()) if last_loss is not None else 0.0,
               "tokens_seen": trainer.tokens_seen, "steps_completed": steps_done}
    if tracker is not None:
      tracker.end_run(run_id, "killed" if stopped else "completed", results)
    return results
  except Exception as e:
    if health is not None:
      health.fail(f"{type(e).__name__}: {e}")
    if tracker is not None:
      tracker.end_run(run_id, "failed")
    raise
  finally:
    stopper.restore()
    profiler.close()
    checkpointer.close()
    metrics.close()
    if tracker is not None:
      tracker.close()
    if trainer.model.rdep is not None:
      trainer.model.rdep.close()


def main(argv: Optional[list] = None) -> None:
  argv = list(sys.argv[1:] if argv is None else argv)
  if not argv or argv[0].startswith("--"):
    raise SystemExit("usage: python -m nmoe_b200.train <config.toml> [--key=value ...]")
  cfg = from_toml(argv[0], argv[1:])
  try:
    train(cfg)
  finally:
    runtime.finalize()


if __name__ == "__main__":
  main()
