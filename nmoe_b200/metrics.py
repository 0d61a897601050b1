"""Metrics: per-rank time-series store, deferred CUDA-event timers, FLOPs model, console line,
router health, GPU telemetry.

Store schema (nmoe/metrics.py:546-597): ``metrics(run TEXT, tag TEXT, step INT, ts_ms BIGINT,
value DOUBLE, PRIMARY KEY(run, tag, step))`` with insert-or-replace semantics, one file per rank at
``{metrics_dir}/{run}/rank_{r}.duckdb``.  DuckDB is used when importable; otherwise the same
table lives in an SQLite file ``rank_{r}.sqlite`` (a dashboard only needs the table).
Tags follow the reference: train/loss, optimizer/lr, throughput/*, efficiency/*, memory/*,
router/layer_NN/*, router_agg/*, time_ms/r{rank}/*, comm/r{rank}/*, gpu/{i}/*, gpu_agg/*.
"""
from __future__ import annotations

import math
import os
import sqlite3
import time
from contextlib import contextmanager, nullcontext
from pathlib import Path
from typing import Dict, Iterable, List, Optional, Tuple

import torch
import torch.distributed as dist

B200_PEAK_TFLOPS = {"bf16": 2250.0, "fp8": 4500.0, "nvfp4": 9000.0, "nvfp4x16": 9000.0}
_SCHEMA = ("CREATE TABLE IF NOT EXISTS metrics (run TEXT, tag TEXT, step INTEGER, ts_ms BIGINT, value DOUBLE, "
           "PRIMARY KEY (run, tag, step))")


class MetricsWriter:
  def __init__(self, run: str, metrics_dir: str, rank: int):
    self.run = run
    d = Path(metrics_dir) / run
    d.mkdir(parents=True, exist_ok=True)
    self.kind = "sqlite"
    try:
      import duckdb  # type: ignore
      self.db = duckdb.connect(str(d / f"rank_{rank}.duckdb"))
      self.kind = "duckdb"
    except ImportError:
      self.db = sqlite3.connect(str(d / f"rank_{rank}.sqlite"), timeout=30.0)
      self.db.execute("PRAGMA journal_mode=WAL")
    self.db.execute(_SCHEMA)
    self.path = d

  def insert_many(self, step: int, items: Iterable[Tuple[str, float]]) -> None:
    ts = int(time.time() * 1000)
    rows = [(self.run, tag, int(step), ts, float(v)) for tag, v in items if v is not None and math.isfinite(float(v))]
    if not rows:
      return
    self.db.executemany("INSERT OR REPLACE INTO metrics VALUES (?, ?, ?, ?, ?)", rows)
    if self.kind == "sqlite":
      self.db.commit()

  def query(self, tag: str) -> List[Tuple[int, float]]:
    cur = self.db.execute("SELECT step, value FROM metrics WHERE run = ? AND tag = ? ORDER BY step", (self.run, tag))
    return [(int(s), float(v)) for s, v in cur.fetchall()]

  def close(self) -> None:
    try:
      self.db.close()
    except Exception:
      pass


class EventTimers:
  """``with timers.time(tag)`` records two CUDA events on the current stream; durations are read
  later with ``event.query()`` so the training thread never blocks on them."""

  def __init__(self, enabled: bool):
    self.enabled = enabled and torch.cuda.is_available()
    self.pending: List[Tuple[str, torch.cuda.Event, torch.cuda.Event]] = []
    self.cpu: List[Tuple[str, float]] = []

  @contextmanager
  def time(self, tag: str):
    if not self.enabled:
      t0 = time.perf_counter()
      yield
      self.cpu.append((tag, (time.perf_counter() - t0) * 1e3))
      return
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    yield
    b.record()
    self.pending.append((tag, a, b))

  def drain(self) -> Dict[str, float]:
    """Mean ms per tag over the intervals that have completed; unfinished ones stay queued."""
    sums: Dict[str, List[float]] = {}
    keep = []
    for tag, a, b in self.pending:
      if b.query():
        sums.setdefault(tag, []).append(a.elapsed_time(b))
      else:
        keep.append((tag, a, b))
    self.pending = keep
    for tag, ms in self.cpu:
      sums.setdefault(tag, []).append(ms)
    self.cpu = []
    return {k: sum(v) / len(v) for k, v in sums.items()}


def param_counts(model, cfg, world: int = 1) -> Tuple[int, int]:
  """(parameters of the whole model, parameters a token touches).  Routed experts are rank-local, so the job holds
  ``world`` times what this rank sees; a token uses ``n_activated_experts`` of ``n_routed_experts`` of them
  (nmoe/metrics.py:384-421)."""
  experts, dense = model.param_sets() if hasattr(model, "param_sets") else ([], list(model.parameters()))
  n_exp = sum(p.numel() for p in experts) * max(1, world)
  n_dense = sum(p.numel() for p in dense)
  frac = cfg.n_activated_experts / cfg.n_routed_experts if getattr(cfg, "n_routed_experts", 0) else 0.0
  return n_dense + n_exp, n_dense + int(n_exp * frac)


def param_summary(model, cfg, world: int = 1) -> str:
  total, active = param_counts(model, cfg, world)
  return f"({total / 1e9:.2f}B params {active / 1e9:.2f}B active)"


def flops_per_token(cfg, seq_len: Optional[int] = None) -> float:
  """6 * (active non-embedding params) + 6 * L * heads * (nope + rope + v) * seq (nmoe/metrics.py:69-124)."""
  S = seq_len or cfg.seq_len
  H, L = cfg.dim, cfg.n_layers
  attn = (H * cfg.q_lora_rank + cfg.q_lora_rank * cfg.n_heads * cfg.qk_head_dim
          + H * (cfg.kv_lora_rank + cfg.qk_rope_head_dim)
          + cfg.kv_lora_rank * cfg.n_heads * (cfg.qk_nope_head_dim + cfg.v_head_dim) + cfg.n_heads * cfg.v_head_dim * H)
  dense = L * attn + cfg.n_dense_layers * 3 * H * (cfg.inter_dim or 0) + cfg.vocab_size * H
  l_moe = max(0, L - cfg.n_dense_layers)
  moe = 0
  if cfg.has_moe:
    F = cfg.moe_inter_dim or cfg.inter_dim
    moe = l_moe * (H * cfg.n_routed_experts + cfg.n_activated_experts * 3 * H * F + cfg.n_shared_experts * 3 * H * F)
  return 6.0 * (dense + moe) + 6.0 * L * cfg.n_heads * (cfg.qk_nope_head_dim + cfg.qk_rope_head_dim + cfg.v_head_dim) * S


def router_stats(loads: torch.Tensor, biases: Optional[List[torch.Tensor]] = None) -> List[Dict[str, float]]:
  """Per MoE layer: cv, entropy, experts_active, max_load (fraction), bias_range.  loads: [L, E] counts."""
  out = []
  frac = loads.float() / loads.float().sum(-1, keepdim=True).clamp_min(1.0)
  for i in range(frac.size(0)):
    f = frac[i]
    mean = f.mean().item()
    cv = (f.std(unbiased=False).item() / mean) if mean > 0 else 0.0
    ent = float(-(f[f > 0] * f[f > 0].log()).sum().item())
    d = {"cv": cv, "entropy": ent, "experts_active": float((f > 0).sum().item()), "max_load": float(f.max().item())}
    if biases is not None:
      b = biases[i]
      d["bias_range"] = float((b.max() - b.min()).item())
      d["bias_min"], d["bias_max"] = float(b.min().item()), float(b.max().item())
    out.append(d)
  return out


# The timers of the running session, for code below the training loop (ZeRO-2, expert dispatch / return) that wants
# to time a span without being handed the session: ``with span("time_ms/zero2_reduce_scatter"): ...``
_ACTIVE_TIMERS: Optional[EventTimers] = None


def span(tag: str):
  """Time a span under ``tag`` in the running metrics session; a no-op context when there is none."""
  t = _ACTIVE_TIMERS
  return t.time(tag) if t is not None else nullcontext()


def register_model_timers(model: torch.nn.Module, timers: EventTimers) -> int:
  """Forward / backward timers on the model's building blocks, without touching model code: module hooks record CUDA
  events on the current stream, the durations are collected when the log line is written (nmoe/metrics.py:276-349 times
  the dense MLP and the head this way; here attention, the MoE layer and the shared / dense MLPs are covered too).
  Tags: time_ms/{attn,moe,dense_mlp}_{fwd,bwd}.  Returns the number of modules hooked."""
  if not timers.enabled:
    return 0
  from .models.mlp import MLP
  from .models.moe import MoE
  n = 0

  def install(mod: torch.nn.Module, tag: str) -> None:
    slot = {}

    def fwd_pre(_m, _inp):
      ev = torch.cuda.Event(enable_timing=True)
      ev.record()
      slot["f"] = ev

    def fwd_post(_m, _inp, _out):
      ev = torch.cuda.Event(enable_timing=True)
      ev.record()
      if "f" in slot:
        timers.pending.append((f"time_ms/{tag}_fwd", slot.pop("f"), ev))

    def bwd_pre(_m, _g):
      ev = torch.cuda.Event(enable_timing=True)
      ev.record()
      slot["b"] = ev

    def bwd_post(_m, _gi, _go):
      ev = torch.cuda.Event(enable_timing=True)
      ev.record()
      if "b" in slot:
        timers.pending.append((f"time_ms/{tag}_bwd", slot.pop("b"), ev))

    mod.register_forward_pre_hook(fwd_pre)
    mod.register_forward_hook(fwd_post)
    mod.register_full_backward_pre_hook(bwd_pre)
    mod.register_full_backward_hook(bwd_post)

  for blk in getattr(model, "blocks", []):
    if hasattr(blk, "attn"):
      install(blk.attn, "attn"); n += 1
    ffn = getattr(blk, "ffn", None)
    if isinstance(ffn, MoE):
      install(ffn, "moe"); n += 1
    elif isinstance(ffn, MLP):
      install(ffn, "dense_mlp"); n += 1
  return n


class MetricsSession:
  def __init__(self, run: str, metrics_dir: str, rank: int, world: int, model, cfg):
    self.run, self.rank, self.world, self.cfg = run, rank, world, cfg
    self.writer: Optional[MetricsWriter] = None
    try:
      self.writer = MetricsWriter(run, os.environ.get("NMOE_METRICS_DIR", metrics_dir), rank)
    except OSError as e:
      if rank == 0:
        print(f"[metrics] store disabled: {e}", flush=True)
    self.timers = EventTimers(os.environ.get("NMOE_TIMERS", "1") not in ("0", "false", "False"))
    global _ACTIVE_TIMERS
    _ACTIVE_TIMERS = self.timers
    # per-module hooks break the block-level activation checkpointing's assumptions about module outputs only in
    # "full" mode, where a block is re-run inside backward; they are installed for the other modes
    if model is not None and getattr(cfg, "activation_checkpoint", "none") != "full" \
        and os.environ.get("NMOE_MODULE_TIMERS", "1") not in ("0", "false", "False"):
      register_model_timers(model, self.timers)
    self.fpt = flops_per_token(cfg)
    self.t_last = time.perf_counter()
    self.step_last = 0
    self.gpu = None
    if rank == 0:
      try:
        from .utils.gpu_telemetry import GpuPoller
        self.gpu = GpuPoller(interval_ms=1000)
        self.gpu.start()
      except Exception:
        self.gpu = None

  def timer(self, tag: str):
    return self.timers.time(tag)

  def insert_many(self, step: int, items) -> None:
    if self.writer is not None:
      self.writer.insert_many(step, items)

  def close(self) -> None:
    global _ACTIVE_TIMERS
    if _ACTIVE_TIMERS is self.timers:
      _ACTIVE_TIMERS = None
    if self.gpu is not None:
      self.gpu.stop()
    if self.writer is not None:
      self.writer.close()


def log_training_step(ms: MetricsSession, step: int, trainer, loss: torch.Tensor, loader_wait_ms: float,
                      print_fn=print) -> None:
  """Every ``log_every`` steps: reduce loss / grad norm, write the time series, print the console line
  ``step loss grad_norm memory tps tflops ms/step node_tps`` (nmoe/metrics.py:480-495)."""
  cfg = ms.cfg
  if step % cfg.log_every != 0 and step != 1:
    return
  lv = loss.detach().float().clone()
  if dist.is_initialized() and ms.world > 1:
    dist.all_reduce(lv)
    lv /= ms.world
  gn = trainer.grad_norm() if trainer.track_gradnorm else None
  if torch.cuda.is_available():
    torch.cuda.synchronize()
  now = time.perf_counter()
  n_steps = max(1, step - ms.step_last)
  dt = max(1e-9, now - ms.t_last)
  ms.t_last, ms.step_last = now, step
  tokens_gpu = cfg.batch_size * cfg.seq_len / ms.world
  tps = tokens_gpu * n_steps / dt
  tflops = tps * ms.fpt / 1e12
  mem_cur = torch.cuda.memory_allocated() / 2 ** 30 if torch.cuda.is_available() else 0.0
  mem_max = torch.cuda.max_memory_allocated() / 2 ** 30 if torch.cuda.is_available() else 0.0
  items = [("train/loss", lv.item()), ("optimizer/lr", trainer.lr), ("throughput/tokens_per_s_gpu", tps),
           ("throughput/ms_per_step", dt / n_steps * 1e3), ("throughput/loader_wait_ms", loader_wait_ms),
           (f"throughput/r{ms.rank}/tokens_per_s", tps), ("efficiency/tflops", tflops),
           (f"efficiency/{cfg.dtype}_tflops", tflops), ("memory/current_alloc_gib", mem_cur),
           ("memory/max_alloc_gib", mem_max), ("health/heartbeat", time.time())]
  if gn is not None:
    items.append(("train/grad_norm", gn.item()))
  for tag, v in ms.timers.drain().items():
    items.append((tag.replace("time_ms/", f"time_ms/r{ms.rank}/"), v))
  rdep = getattr(trainer.model, "rdep", None)
  if rdep is not None and hasattr(rdep, "comm_counters"):
    items += [(f"comm/r{ms.rank}/{k}", v) for k, v in rdep.comm_counters().items()]
  rs_line = ""
  loads = trainer.model.expert_loads() if hasattr(trainer.model, "expert_loads") else None
  if loads is not None:
    biases = [m.router.bias for m in trainer.model.moe_layers()]
    stats = router_stats(loads, biases)
    for i, s in enumerate(stats):
      for k in ("cv", "entropy", "experts_active", "bias_range", "max_load"):
        items.append((f"router/layer_{i:02d}/{k}", s[k]))
    agg_cv = sum(s["cv"] for s in stats) / len(stats)
    agg_max = max(s["max_load"] for s in stats)
    bmin, bmax = min(s["bias_min"] for s in stats), max(s["bias_max"] for s in stats)
    items += [("router_agg/mean_cv", agg_cv), ("router_agg/max_load", agg_max),
              ("router_agg/dead_experts", sum(cfg.n_routed_experts - s["experts_active"] for s in stats))]
    rs_line = f" | router: cv {agg_cv:.3f} max {agg_max:.4f} bias[{bmin:+.4f},{bmax:+.4f}]"
  if ms.gpu is not None:
    from .utils.gpu_telemetry import dashboard_items
    items += dashboard_items(ms.gpu.snapshot())
  ms.insert_many(step, items)
  gn_s = f"{gn.item():.3f}" if gn is not None else "-"
  print_fn(f"step {step:>6} loss {lv.item():.4f} grad_norm {gn_s} memory {mem_max:.1f}GiB tps {tps:,.0f} "
           f"tflops {tflops:.1f} ms/step {dt / n_steps * 1e3:.1f} node_tps {tps * ms.world:,.0f}{rs_line}")
