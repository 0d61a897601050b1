"""Split checkpoints with asynchronous writes, atomic finalisation and exact resume.

Layout (same as the reference, nmoe/checkpoint.py:19-795):
  {dir}/latest_checkpointed_iteration.txt        last finalised step (tmp + replace + fsync)
  {dir}/iter_{step:07d}/rd.pt                    rank 0: step, tokens, config_fingerprint, model_dense,
                                                 run_info, plan_bundle
  {dir}/iter_{step:07d}/dp_rank_{rank:03d}.pt    every rank: step, model_expert (W1/W3/W2 of the local
                                                 experts in the reference layout), optimizer (expert
                                                 AdamW state), loader cursors, RNG state, zero2 shard
                                                 state, config_fingerprint
  {dir}/iter_{step:07d}/manifest.json            {step, world, dp_count, bytes_total, git_sha, files}
A step counts as saved only once its manifest exists and the tracker points at it; a crash
between files leaves the previous step as the latest.  Tensors are copied to host memory
synchronously at ``submit`` (so training may overwrite them), serialisation and fsync happen on
a writer thread whose first error is latched and re-raised on the next submit/wait/close.  A
purger keeps the newest ``keep_last`` finalised steps.  Resume refuses a different config
fingerprint, mixture-plan hash or world size.
"""
from __future__ import annotations

import json
import math
import os
import queue
import shutil
import subprocess
import threading
import time
from pathlib import Path
from typing import Any, Callable, Dict, Optional, Tuple

import torch

from .config import Config, fingerprint
from .parallel.rdep import from_reference_layout, to_reference_layout

TRACKER = "latest_checkpointed_iteration.txt"


def iteration_dir(base: str | Path, step: int) -> Path:
  return Path(base) / f"iter_{step:07d}"


def _fsync_dir(path: Path) -> None:
  try:
    fd = os.open(str(path), os.O_RDONLY)
    try:
      os.fsync(fd)
    finally:
      os.close(fd)
  except OSError:
    pass


def atomic_write_text(path: Path, text: str) -> None:
  path.parent.mkdir(parents=True, exist_ok=True)
  tmp = path.with_name(path.name + f".tmp.{os.getpid()}.{threading.get_ident()}")
  with open(tmp, "w") as f:
    f.write(text)
    f.flush()
    os.fsync(f.fileno())
  os.replace(tmp, path)
  _fsync_dir(path.parent)


def read_tracker(base: str | Path) -> int:
  try:
    return int((Path(base) / TRACKER).read_text().strip())
  except (OSError, ValueError):
    return -1


def read_latest_run_info(base: str | Path) -> Optional[dict]:
  """``run_info`` of the latest finalised step (git hash, preset, dtype, expert count, ...) plus ``step`` and ``tokens``,
  read from ``rd.pt`` on the CPU; None when there is no readable checkpoint (nmoe/checkpoint.py:80-101)."""
  step = read_tracker(base)
  if step < 0:
    return None
  try:
    rd = torch.load(iteration_dir(base, step) / "rd.pt", map_location="cpu", weights_only=False)
  except (OSError, RuntimeError, EOFError, ValueError):
    return None
  info = rd.get("run_info")
  if not isinstance(info, dict):
    return None
  return {**info, "step": int(rd.get("step", step)), "tokens": int(rd.get("tokens", 0))}


def git_sha() -> str:
  try:
    return subprocess.run(["git", "rev-parse", "HEAD"], capture_output=True, text=True, timeout=5,
                          cwd=Path(__file__).resolve().parent).stdout.strip() or "unknown"
  except (OSError, subprocess.SubprocessError):
    return "unknown"


def to_host(obj: Any) -> Any:
  """Deep copy of a nested state with every tensor on the CPU."""
  if isinstance(obj, torch.Tensor):
    return obj.detach().to("cpu", copy=True)
  if isinstance(obj, dict):
    return {k: to_host(v) for k, v in obj.items()}
  if isinstance(obj, (list, tuple)):
    return type(obj)(to_host(v) for v in obj)
  return obj


def try_finalize_step(base: str | Path, step: int, world: int) -> bool:
  """Write the manifest and flip the tracker once rd.pt and all ``world`` dp files exist."""
  d = iteration_dir(base, step)
  files = [d / "rd.pt"] + [d / f"dp_rank_{r:03d}.pt" for r in range(world)]
  if not all(f.exists() for f in files):
    return False
  manifest = {"step": step, "world": world, "dp_count": world, "git_sha": git_sha(),
              "bytes_total": sum(f.stat().st_size for f in files), "files": [f.name for f in files]}
  atomic_write_text(d / "manifest.json", json.dumps(manifest, indent=1, sort_keys=True))
  if read_tracker(base) < step:
    atomic_write_text(Path(base) / TRACKER, str(int(step)))
  return True


class Checkpointer:
  def __init__(self, base: str, keep_last: int = 3, async_io: bool = True, async_max_queue: int = 1,
               fault_hook: Optional[Callable[[str], None]] = None):
    """``fault_hook(stage)`` is called at 'before_write', 'after_write', 'before_finalize'; tests use it to
    simulate a crash between files."""
    self.base = Path(base)
    self.keep_last = int(keep_last)
    self.async_io = async_io
    self.fault_hook = fault_hook
    self._err: Optional[BaseException] = None
    self.last_write_ms = 0.0      # serialise + fsync + finalise of the newest file written, measured on the writer
    self.last_stage_ms = 0.0      # device -> host copy of the newest submit, measured on the training thread
    self._q: "queue.Queue[Optional[Tuple[Path, dict, int, int]]]" = queue.Queue(maxsize=max(1, async_max_queue))
    self._thread: Optional[threading.Thread] = None
    if async_io:
      self._thread = threading.Thread(target=self._run, name="ckpt-writer", daemon=True)
      self._thread.start()

  # ---------------------------------------------------------------- writer
  def _write(self, path: Path, state: dict, step: int, world: int) -> None:
    t0 = time.perf_counter()
    if self.fault_hook:
      self.fault_hook("before_write")
    path.parent.mkdir(parents=True, exist_ok=True)
    tmp = path.with_name(path.name + ".tmp")
    with open(tmp, "wb") as f:
      torch.save(state, f)
      f.flush()
      os.fsync(f.fileno())
    os.replace(tmp, path)
    _fsync_dir(path.parent)
    if self.fault_hook:
      self.fault_hook("after_write")
      self.fault_hook("before_finalize")
    if try_finalize_step(self.base, step, world):
      self._purge()
    self.last_write_ms = (time.perf_counter() - t0) * 1e3

  def recommend_interval(self, step_time_ms: float, safety: float = 1.3) -> int:
    """The smallest ``checkpoint_every`` at which the asynchronous writer keeps up: a save must be on disk before the
    next one is submitted, or ``submit`` blocks the training loop on the queue.  1 until a save has been timed
    (nmoe/checkpoint.py:534-541)."""
    if self.last_write_ms <= 0 or step_time_ms <= 0:
      return 1
    return max(1, math.ceil(safety * self.last_write_ms / step_time_ms))

  def _run(self) -> None:
    while True:
      task = self._q.get()
      try:
        if task is None:
          return
        if self._err is None:
          self._write(*task)
      except BaseException as e:  # latched; surfaced on the training thread
        self._err = e
      finally:
        self._q.task_done()

  def _raise_if_failed(self) -> None:
    if self._err is not None:
      e, self._err = self._err, None
      raise RuntimeError(f"asynchronous checkpoint write failed: {e!r}") from e

  def submit(self, path: Path, state: dict, step: int, world: int) -> None:
    self._raise_if_failed()
    t0 = time.perf_counter()
    host = to_host(state)
    self.last_stage_ms = (time.perf_counter() - t0) * 1e3
    if self.async_io:
      self._q.put((path, host, step, world))
    else:
      self._write(path, host, step, world)

  def wait(self) -> None:
    if self.async_io:
      self._q.join()
    self._raise_if_failed()

  def close(self) -> None:
    if self._thread is not None:
      self._q.join()
      self._q.put(None)
      self._thread.join(timeout=60)
      self._thread = None
    self._raise_if_failed()

  # ---------------------------------------------------------------- retention / discovery
  def _finalized_steps(self) -> list[int]:
    out = []
    for d in self.base.glob("iter_*"):
      if (d / "manifest.json").exists():
        try:
          out.append(int(d.name.split("_")[1]))
        except ValueError:
          pass
    return sorted(out)

  def _purge(self) -> None:
    if self.keep_last <= 0:
      return
    steps = self._finalized_steps()
    latest = read_tracker(self.base)
    for s in steps[:-self.keep_last]:
      if s != latest:
        shutil.rmtree(iteration_dir(self.base, s), ignore_errors=True)

  def find_latest(self, rank: int) -> int:
    """Newest step that is finalised and has this rank's file; -1 if none."""
    cands = [s for s in self._finalized_steps() if (iteration_dir(self.base, s) / f"dp_rank_{rank:03d}.pt").exists()]
    t = read_tracker(self.base)
    cands = [s for s in cands if s <= t] if t >= 0 else []
    return cands[-1] if cands else -1


# -------------------------------------------------------------------- state assembly
def _expert_names(model) -> Dict[str, Tuple[Any, int]]:
  return {f"blocks.{b.layer_id}.ffn": b.ffn for b in model.blocks if getattr(b, "is_moe", False)}


def build_states(step: int, trainer, loader, plan, cfg: Config, rank: int, world: int, fp: str):
  model = trainer.model
  expert_param_ids = {id(p) for p in model.param_sets()[0]}
  dense = {k: v for k, v in model.state_dict().items()
           if not any(k == n for n, p in model.named_parameters() if id(p) in expert_param_ids)}
  rd = None
  if rank == 0:
    rd = {"step": step, "tokens": trainer.tokens_seen, "config_fingerprint": fp, "model_dense": dense,
          "run_info": {"git_sha": git_sha(), "preset": cfg.preset, "dtype": cfg.dtype, "E": cfg.n_routed_experts,
                       "K": cfg.n_activated_experts, "H": cfg.dim, "L": cfg.n_layers, "world": world,
                       "dataset_version": getattr(plan, "plan_id", None), "tokenizer_id": cfg.tokenizer}}
    if plan is not None:
      rd["plan_bundle"] = {"mixture_id": plan.mixture_id, "flow_mode": plan.flow_mode, "plan_hash": plan.plan_hash,
                           "plan_json": plan.to_json()}
  experts = {}
  for name, moe in _expert_names(model).items():
    W1, W3, W2 = to_reference_layout(moe.W13.data, moe.W2.data)
    experts[name + ".W1"], experts[name + ".W3"], experts[name + ".W2"] = W1, W3, W2
  rng = {"torch": torch.get_rng_state()}
  if torch.cuda.is_available():
    rng["cuda"] = torch.cuda.get_rng_state_all()
  dp = {"step": step, "tokens": trainer.tokens_seen, "model_expert": experts,
        "optimizer": trainer.opt.expert.state_dict() if trainer.opt.expert is not None else None,
        "loader": loader.state_dict() if loader is not None else None, "rng": rng, "config_fingerprint": fp,
        "zero2": trainer.opt.dense.state_dict(), "world": world}
  return rd, dp


def save_checkpoint(ck: Checkpointer, step: int, trainer, loader, plan, cfg: Config, rank: int, fp: str,
                    print_fn=print, force: bool = False) -> bool:
  if not (force or step % max(1, cfg.checkpoint_every) == 0 or step == cfg.steps):
    return False
  world = trainer.world
  # a bounded wait that ran out, or rows dropped by a full receive buffer, means some rank trained on stale or
  # incomplete data: no rank may turn that state into a checkpoint
  from .ops import tc_gemm
  tc_gemm.check_status_collective(trainer.device, world)
  rd, dp = build_states(step, trainer, loader, plan, cfg, rank, world, fp)
  d = iteration_dir(ck.base, step)
  if rd is not None:
    ck.submit(d / "rd.pt", rd, step, world)
  ck.submit(d / f"dp_rank_{rank:03d}.pt", dp, step, world)
  note = ""
  if ck.last_write_ms > 0:
    note = f" (host copy {ck.last_stage_ms:.0f} ms; previous write {ck.last_write_ms / 1e3:.1f} s)"
  print_fn(f"[ckpt] step {step} submitted -> {d}{note}")
  return True


def load_checkpoint(ck: Checkpointer, trainer, loader, plan, cfg: Config, rank: int, print_fn=print) -> Tuple[int, int]:
  """Restore the newest finalised step.  Returns (start_step, tokens_seen); (0, 0) when starting fresh."""
  if not cfg.resume:
    return 0, 0
  step = ck.find_latest(rank)
  if step < 0:
    return 0, 0
  d = iteration_dir(ck.base, step)
  rd = torch.load(d / "rd.pt", map_location="cpu", weights_only=False)
  dp = torch.load(d / f"dp_rank_{rank:03d}.pt", map_location="cpu", weights_only=False)
  fp = fingerprint(cfg)
  for what, state in (("rd.pt", rd), ("dp file", dp)):
    if state.get("config_fingerprint") != fp:
      raise RuntimeError(f"refusing to resume from {d}: config fingerprint of {what} differs from the current config "
                         "(set resume=false or use a new checkpoint_dir)")
  if int(dp.get("world", trainer.world)) != trainer.world:
    raise RuntimeError(f"checkpoint was written with world={dp['world']}, now {trainer.world}: ZeRO-2 shards and "
                       "expert placement are tied to the world size")
  if plan is not None and "plan_bundle" in rd and rd["plan_bundle"]["plan_hash"] != plan.plan_hash:
    raise RuntimeError("refusing to resume: data mixture plan hash changed")
  model = trainer.model
  missing, unexpected = model.load_state_dict(rd["model_dense"], strict=False)
  expert_keys = {n for n, p in model.named_parameters() if id(p) in {id(q) for q in model.param_sets()[0]}}
  bad = [k for k in missing if k not in expert_keys]
  if bad or unexpected:
    raise RuntimeError(f"dense state mismatch: missing={bad} unexpected={list(unexpected)}")
  with torch.no_grad():
    for name, moe in _expert_names(model).items():
      e = dp["model_expert"]
      W13, W2 = from_reference_layout(e[name + ".W1"], e[name + ".W3"], e[name + ".W2"])
      moe.W13.data.copy_(W13)
      moe.W2.data.copy_(W2)
  if trainer.opt.expert is not None and dp.get("optimizer") is not None:
    trainer.opt.expert.load_state_dict(dp["optimizer"])
  trainer.opt.dense.load_state_dict(dp["zero2"])
  if loader is not None and dp.get("loader") is not None:
    loader.load_state_dict(dp["loader"])
  torch.set_rng_state(dp["rng"]["torch"])
  if torch.cuda.is_available() and "cuda" in dp["rng"]:
    try:
      torch.cuda.set_rng_state_all(dp["rng"]["cuda"])
    except RuntimeError:
      pass
  print_fn(f"[ckpt] resumed from {d} (step {step}, {int(rd['tokens']):,} tokens)")
  return int(rd["step"]), int(rd["tokens"])
