"""Interactive toolkit: the helpers one reaches for in a notebook or a REPL next to a model.

    from nmoe_b200 import lab
    t = lab.tiny_trainer(n_layers=4)              # or lab.trainer_from("configs/moonlet.toml", steps=50)
    lab.param_memory(t.model)                     # bytes by parameter group
    lab.time_step(t, iters=10)                    # forward / backward / optimizer, device-timed on a GPU
    lab.profile_steps(t, steps=3)                 # top kernels / operators / scopes per step (torch.profiler)
    with lab.RouterProbe(t.model) as probe: lab.run_steps(t, 5)
    probe.table()                                 # per-layer load CV, entropy, dead experts, hottest expert
    lab.grad_report(t.model)                      # gradient norms per block
    lab.peek_checkpoint("/data/checkpoints/run")  # what a checkpoint holds, without loading it
    lab.quick_train({"lr_dense": 3e-3}, steps=20) # a loss curve for a quick ablation

The same ground as the reference's ``notebooks/quickstart.ipynb`` toolkit cells (memory, timing, MoE routing, gradient
health, checkpoints, quick ablations), as an importable and tested module instead of notebook cells.  Everything returns
plain Python data (dicts, lists of rows); ``show`` prints rows as an aligned table, and nothing needs a plotting package.
"""
from __future__ import annotations

import json
import math
import time
from collections import defaultdict
from pathlib import Path
from typing import Any, Dict, List, Optional, Sequence

import torch

from .config import Config, from_toml
from .metrics import router_stats

Row = Dict[str, Any]


# ---------------------------------------------------------------------------------------------- construction
_TINY = dict(vocab_size=512, eos_token_id=511, dim=64, n_layers=2, n_heads=2, inter_dim=128, moe_inter_dim=32,
             n_routed_experts=8, n_activated_experts=2, n_shared_experts=1, n_dense_layers=1, q_lora_rank=32, kv_lora_rank=16,
             qk_nope_head_dim=16, qk_rope_head_dim=8, v_head_dim=16, batch_size=2, seq_len=64, max_position_embeddings=128,
             warmup_steps=2, steps=100, data_path="synthetic", activation_checkpoint="none")


# The same idea at the smallest sizes the GPU kernels take (head dimensions and widths in multiples of their tiles).
_TINY_GPU = dict(vocab_size=2048, eos_token_id=2047, dim=512, n_layers=2, n_heads=4, inter_dim=1024, moe_inter_dim=256,
                 n_routed_experts=8, n_activated_experts=2, n_shared_experts=2, n_dense_layers=1, q_lora_rank=256, kv_lora_rank=128,
                 qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128, batch_size=4, seq_len=256, max_position_embeddings=512,
                 warmup_steps=2, steps=100, data_path="synthetic", activation_checkpoint="none")


def _device() -> torch.device:
  return torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")


def tiny_trainer(fused: bool = False, **overrides):
  """A two-layer model that steps in milliseconds: for trying the tools below, and for tests.  On a GPU the sizes are
  the smallest the kernels take (``_TINY_GPU``), on a CPU smaller still.

  ``fused=False`` keeps the expert optimizer out of backward, so that expert gradients are there to look at after
  ``backward_only`` and a backward pass changes no weight; ``fused=True`` is what training does."""
  from .train import Trainer
  dev = _device()
  cfg = Config(**{**(_TINY_GPU if dev.type == "cuda" else _TINY), **overrides})
  cfg.validate(1)
  torch.manual_seed(cfg.seed)
  return Trainer(cfg, device=dev, fuse_expert_opt=fused)


def trainer_from(config_path: str, fused: bool = False, **overrides):
  """A single-process trainer for a configuration file with ``key=value`` overrides (``fused``: see ``tiny_trainer``)."""
  from .train import Trainer
  cfg = from_toml(config_path, [f"--{k}={v}" for k, v in overrides.items()], env={})
  cfg.validate(1)
  torch.manual_seed(cfg.seed)
  return Trainer(cfg, device=_device(), fuse_expert_opt=fused)


def random_batch(cfg: Config, device=None, seed: int = 0):
  g = torch.Generator().manual_seed(seed)
  x = torch.randint(0, cfg.vocab_size, (cfg.batch_size, cfg.seq_len + 1), generator=g)
  dev = device or _device()
  return x[:, :-1].contiguous().to(dev), x[:, 1:].contiguous().to(dev)


def run_steps(trainer, n: int, batch=None) -> List[float]:
  """``n`` optimizer steps on one fixed random batch (the loss must fall); returns the losses."""
  x, y = batch or random_batch(trainer.cfg, trainer.device)
  return [float(trainer.step(x, y)) for _ in range(n)]


# ---------------------------------------------------------------------------------------------- tables
def show(rows: Sequence[Row], columns: Optional[Sequence[str]] = None, print_fn=print) -> str:
  """Rows as an aligned text table; returns the text as well as printing it."""
  if not rows:
    print_fn("(no rows)")
    return ""
  cols = list(columns or rows[0].keys())
  def cell(v):
    if isinstance(v, float):
      return f"{v:.4g}"
    return str(v)
  body = [[cell(r.get(c, "")) for c in cols] for r in rows]
  width = [max(len(c), *(len(b[i]) for b in body)) for i, c in enumerate(cols)]
  lines = ["  ".join(c.ljust(w) for c, w in zip(cols, width)), "  ".join("-" * w for w in width)]
  lines += ["  ".join(v.rjust(w) if _is_num(v) else v.ljust(w) for v, w in zip(b, width)) for b in body]
  text = "\n".join(lines)
  print_fn(text)
  return text


def _is_num(s: str) -> bool:
  try:
    float(s)
    return True
  except ValueError:
    return False


# ---------------------------------------------------------------------------------------------- memory
def mem_stats(device=None) -> Dict[str, float]:
  """Allocator state in GiB (zeros on a machine without a GPU)."""
  if not torch.cuda.is_available():
    return {"allocated_gib": 0.0, "reserved_gib": 0.0, "peak_gib": 0.0, "free_gib": 0.0, "total_gib": 0.0}
  gib = float(1 << 30)
  free, total = torch.cuda.mem_get_info(device)
  return {"allocated_gib": torch.cuda.memory_allocated(device) / gib, "reserved_gib": torch.cuda.memory_reserved(device) / gib,
          "peak_gib": torch.cuda.max_memory_allocated(device) / gib, "free_gib": free / gib, "total_gib": total / gib}


def _group_of(name: str) -> str:
  leaf = name.rsplit(".", 1)[-1]
  if leaf in ("W13", "W2"):
    return "routed experts"
  if name in ("embedding", "lm_head"):
    return "embeddings"
  if "norm" in name:
    return "norms"
  if ".attn." in name:
    return "attention"
  if ".router." in name:
    return "router"
  if ".shared." in name:
    return "shared experts"
  return "dense mlp / other"


def param_memory(model: torch.nn.Module) -> List[Row]:
  """Parameter count and bytes by group, largest first, with a total row."""
  acc: Dict[str, List[int]] = defaultdict(lambda: [0, 0, 0])
  for name, p in model.named_parameters():
    a = acc[_group_of(name)]
    a[0] += 1
    a[1] += p.numel()
    a[2] += p.numel() * p.element_size()
  rows = [{"group": g, "tensors": a[0], "params_m": a[1] / 1e6, "mib": a[2] / float(1 << 20)} for g, a in acc.items()]
  rows.sort(key=lambda r: -r["mib"])
  rows.append({"group": "total", "tensors": sum(r["tensors"] for r in rows), "params_m": sum(r["params_m"] for r in rows),
               "mib": sum(r["mib"] for r in rows)})
  return rows


def count_params(cfg: Config) -> Dict[str, int]:
  """Parameter counts from the configuration alone (MLA attention): routed experts, and everything else."""
  H, L = cfg.dim, cfg.n_layers
  attn = (H * cfg.q_lora_rank + cfg.q_lora_rank * cfg.n_heads * (cfg.qk_nope_head_dim + cfg.qk_rope_head_dim)
          + H * (cfg.kv_lora_rank + cfg.qk_rope_head_dim) + cfg.kv_lora_rank * cfg.n_heads * (cfg.qk_nope_head_dim + cfg.v_head_dim)
          + cfg.n_heads * cfg.v_head_dim * H + cfg.q_lora_rank + cfg.kv_lora_rank)
  F = cfg.moe_inter_dim or cfg.inter_dim or 0
  l_moe = max(0, L - cfg.n_dense_layers) if cfg.has_moe else 0
  dense = (L * (attn + 2 * H) + (L - l_moe) * 3 * H * (cfg.inter_dim or 0) + 2 * cfg.vocab_size * H + H
           + l_moe * (H * cfg.n_routed_experts + cfg.n_shared_experts * 3 * H * F))
  return {"dense": int(dense), "expert": int(l_moe * cfg.n_routed_experts * 3 * H * F)}


def training_state_estimate(cfg: Config, world: int = 1) -> Dict[str, float]:
  """GiB per GPU that do not depend on the batch: bf16 weights and gradients, fp32 master copies and AdamW moments
  (12 bytes per parameter).  Dense optimizer state is sharded over the data-parallel group (ZeRO-2); the routed
  experts, with their gradients and optimizer state, are split over the expert-parallel group (the same ranks)."""
  n = count_params(cfg)
  dense, expert = n["dense"], n["expert"]
  gib = float(1 << 30)
  w = max(1, world)
  out = {
    "dense_weights_gib": dense * 2 / gib, "dense_grads_gib": dense * 2 / gib, "dense_opt_gib": dense * 12 / w / gib,
    "expert_weights_gib": expert * 2 / w / gib, "expert_grads_gib": expert * 2 / w / gib, "expert_opt_gib": expert * 12 / w / gib,
  }
  out["total_gib"] = sum(out.values())
  return out


# ---------------------------------------------------------------------------------------------- timing
class _Clock:
  """CUDA events on a GPU, the host clock otherwise; ``ms()`` after ``stop()``."""

  def __init__(self, device: torch.device):
    self.cuda = device.type == "cuda"
    if self.cuda:
      self.a, self.b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

  def start(self):
    if self.cuda:
      self.a.record()
    else:
      self.t = time.perf_counter()

  def stop(self):
    if self.cuda:
      self.b.record()
    else:
      self.dt = (time.perf_counter() - self.t) * 1e3

  def ms(self) -> float:
    if self.cuda:
      self.b.synchronize()
      return self.a.elapsed_time(self.b)
    return self.dt


def time_step(trainer, warmup: int = 3, iters: int = 10, batch=None) -> Dict[str, float]:
  """Mean milliseconds of forward, backward and optimizer step, timed separately, and tokens per second.
  Timing the phases apart serialises work that a training step overlaps (expert optimizer inside backward, ZeRO-2
  buckets): ``total_ms`` here is an upper bound of ``Trainer.step`` time, which ``bench.py`` measures."""
  x, y = batch or random_batch(trainer.cfg, trainer.device)
  m, opt, dev = trainer.model, trainer.opt, trainer.device
  acc = {"forward_ms": 0.0, "backward_ms": 0.0, "optimizer_ms": 0.0}
  for it in range(warmup + iters):
    clocks = {k: _Clock(dev) for k in acc}
    opt.begin_step(trainer.step_num, trainer.tokens_seen, None)
    clocks["forward_ms"].start(); loss = m.loss(x, y); clocks["forward_ms"].stop()
    clocks["backward_ms"].start(); loss.backward(); clocks["backward_ms"].stop()
    clocks["optimizer_ms"].start(); opt.step(); clocks["optimizer_ms"].stop()
    trainer.step_num += 1
    if it >= warmup:
      for k in acc:
        acc[k] += clocks[k].ms()
  out = {k: v / iters for k, v in acc.items()}
  out["total_ms"] = sum(out.values())
  out["tokens_per_s"] = trainer.cfg.batch_size * trainer.cfg.seq_len / (out["total_ms"] / 1e3)
  return out


def profile_steps(trainer, steps: int = 3, warmup: int = 2, top: int = 25, batch=None) -> List[Row]:
  """``steps`` training steps under ``torch.profiler`` with the module scopes on; the ``top`` entries by device time
  (host time without a GPU): kernels, operators and scopes with call counts and milliseconds per step.  For looking at
  a step interactively; kernel counters come from ``ncu`` and throughput from ``bench.py``, never from here."""
  from .utils import profiling as P
  x, y = batch or random_batch(trainer.cfg, trainer.device)
  for _ in range(warmup):
    trainer.step(x, y)
  cuda = trainer.device.type == "cuda"
  acts = [torch.profiler.ProfilerActivity.CPU] + ([torch.profiler.ProfilerActivity.CUDA] if cuda else [])
  P.enable_scopes(True)
  try:
    with torch.profiler.profile(activities=acts) as prof:
      for _ in range(steps):
        trainer.step(x, y)
      if cuda:
        torch.cuda.synchronize(trainer.device)
  finally:
    P.enable_scopes(False)
  rows = []
  for e in prof.key_averages():
    dev_us = float(getattr(e, "self_device_time_total", 0.0) or getattr(e, "self_cuda_time_total", 0.0) or 0.0)
    rows.append({"name": e.key[:70], "calls_per_step": e.count / steps, "device_ms_per_step": dev_us / 1e3 / steps,
                 "host_ms_per_step": float(e.self_cpu_time_total) / 1e3 / steps})
  rows.sort(key=lambda r: -(r["device_ms_per_step"] if cuda else r["host_ms_per_step"]))
  return rows[:top]


# ---------------------------------------------------------------------------------------------- routing
class RouterProbe:
  """Collects the per-layer expert selection counts of every forward pass while active.

  The MoE layers already keep the counts of their last forward (``MoE.loads``, what the training metrics read); the
  probe copies them when the last MoE layer has run, so it adds no work to the layers themselves."""

  def __init__(self, model):
    self.model, self.history, self._h = model, [], None

  def __enter__(self):
    layers = self.model.moe_layers()
    if not layers:
      raise ValueError("the model has no MoE layers")
    def after(_mod, _inp, _out):
      loads = self.model.expert_loads()
      if loads is not None:
        self.history.append(loads.detach().float().cpu())
    self._h = layers[-1].register_forward_hook(after)
    return self

  def __exit__(self, *exc):
    if self._h is not None:
      self._h.remove()
      self._h = None
    return False

  def total(self) -> Optional[torch.Tensor]:
    return torch.stack(self.history).sum(0) if self.history else None

  def table(self) -> List[Row]:
    """Per MoE layer over all recorded passes: load CV, entropy, active experts, hottest expert and its share."""
    tot = self.total()
    if tot is None:
      return []
    rows = []
    for i, s in enumerate(router_stats(tot)):
      frac = tot[i] / tot[i].sum().clamp_min(1.0)
      rows.append({"moe_layer": i, "cv": s["cv"], "entropy": s["entropy"], "experts_active": int(s["experts_active"]),
                   "dead": int(tot.shape[1] - s["experts_active"]), "hottest": int(frac.argmax()), "hottest_share": float(frac.max()),
                   "ideal_share": 1.0 / tot.shape[1]})
    return rows

  def drift(self) -> List[float]:
    """Total-variation distance between the load distributions of consecutive passes, averaged over layers: how fast
    routing is still moving."""
    out = []
    for a, b in zip(self.history, self.history[1:]):
      pa, pb = a / a.sum(-1, keepdim=True).clamp_min(1), b / b.sum(-1, keepdim=True).clamp_min(1)
      out.append(float((pa - pb).abs().sum(-1).mean() / 2))
    return out


# ---------------------------------------------------------------------------------------------- gradients
def _block_of(name: str) -> str:
  parts = name.split(".")
  if parts[0] == "blocks" and len(parts) > 2:
    return f"blocks.{int(parts[1]):02d}.{parts[2]}"
  return parts[0]


def grad_report(model: torch.nn.Module) -> List[Row]:
  """Gradient and weight L2 norms per block (``blocks.NN.attn`` ...), their ratio, and non-finite counts.  Call after
  a backward pass and before the optimizer clears the gradients."""
  acc: Dict[str, List[float]] = defaultdict(lambda: [0.0, 0.0, 0, 0])
  for name, p in model.named_parameters():
    a = acc[_block_of(name)]
    a[1] += float(p.detach().float().pow(2).sum())
    if p.grad is None:
      a[3] += 1
      continue
    g = p.grad.detach().float()
    a[0] += float(g.pow(2).sum())
    a[2] += int((~torch.isfinite(g)).sum())
  rows = []
  for block in sorted(acc):
    g2, w2, bad, missing = acc[block]
    rows.append({"block": block, "grad_norm": math.sqrt(g2), "weight_norm": math.sqrt(w2),
                 "ratio": math.sqrt(g2) / math.sqrt(w2) if w2 > 0 else float("nan"), "non_finite": bad, "no_grad": missing})
  return rows


def backward_only(trainer, batch=None) -> float:
  """One forward + backward without an optimizer step, so that ``grad_report`` sees the gradients.  With a trainer
  built with ``fused=True`` the expert optimizer runs inside this backward pass: expert weights move and their
  gradients are reported as ``no_grad``."""
  x, y = batch or random_batch(trainer.cfg, trainer.device)
  trainer.model.zero_grad(set_to_none=True)
  loss = trainer.model.loss(x, y)
  loss.backward()
  return float(loss.detach())


# ---------------------------------------------------------------------------------------------- checkpoints
def list_checkpoints(base) -> List[Row]:
  """Finalised and unfinished steps under a checkpoint directory."""
  from .checkpoint import read_tracker
  base = Path(base)
  if not base.is_dir():
    return []
  latest = read_tracker(base)
  rows = []
  for d in sorted(base.glob("iter_*")):
    man = d / "manifest.json"
    info = json.loads(man.read_text()) if man.exists() else {}
    rows.append({"step": int(d.name.split("_")[1]), "finalised": man.exists(), "latest": int(d.name.split("_")[1]) == latest,
                 "world": info.get("world"), "gib": (info.get("bytes_total") or 0) / float(1 << 30), "git": (info.get("git_sha") or "")[:10],
                 "files": len(list(d.glob("*.pt")))})
  return rows


def _describe(obj: Any, depth: int = 0, max_items: int = 12) -> Any:
  if isinstance(obj, torch.Tensor):
    return f"tensor{list(obj.shape)} {str(obj.dtype).replace('torch.', '')}"
  if isinstance(obj, dict):
    if depth >= 2:
      return f"dict({len(obj)} keys)"
    items = list(obj.items())
    out = {str(k): _describe(v, depth + 1, max_items) for k, v in items[:max_items]}
    if len(items) > max_items:
      out["..."] = f"{len(items) - max_items} more"
    return out
  if isinstance(obj, (list, tuple)):
    return f"{type(obj).__name__}({len(obj)})" if len(obj) > 4 else [_describe(v, depth + 1, max_items) for v in obj]
  if isinstance(obj, (int, float, str, bool)) or obj is None:
    return obj
  return type(obj).__name__


def peek_checkpoint(base, step: Optional[int] = None, rank: int = 0) -> Dict[str, Any]:
  """What a step's files hold (keys, tensor shapes, step / token counters, fingerprint), read on the CPU without
  building a model.  ``step=None`` takes the latest finalised step."""
  from .checkpoint import iteration_dir, read_tracker
  step = read_tracker(base) if step is None else step
  if step < 0:
    raise FileNotFoundError(f"no finalised checkpoint under {base}")
  d = iteration_dir(base, step)
  out: Dict[str, Any] = {"dir": str(d), "step": step}
  man = d / "manifest.json"
  if man.exists():
    out["manifest"] = json.loads(man.read_text())
  for key, f in (("rd", d / "rd.pt"), ("dp_rank", d / f"dp_rank_{rank:03d}.pt")):
    if f.exists():
      state = torch.load(f, map_location="cpu", weights_only=False)
      out[key] = _describe(state)
      if key == "rd" and isinstance(state.get("model_dense"), dict):
        out["dense_params_m"] = sum(v.numel() for v in state["model_dense"].values() if isinstance(v, torch.Tensor)) / 1e6
  return out


# ---------------------------------------------------------------------------------------------- ablations
def quick_train(overrides: Optional[Dict[str, Any]] = None, steps: int = 20, config_path: Optional[str] = None,
                log_every: int = 5, print_fn=print) -> List[float]:
  """A short run from scratch on synthetic tokens with some configuration keys changed; returns the loss per step.
  Two calls with different overrides and the same seed give curves that can be compared point by point."""
  t = trainer_from(config_path, **{**(overrides or {}), "steps": steps}) if config_path else tiny_trainer(**{**(overrides or {}), "steps": steps})
  g = torch.Generator().manual_seed(t.cfg.seed)
  losses = []
  for s in range(steps):
    tok = torch.randint(0, t.cfg.vocab_size, (t.cfg.batch_size, t.cfg.seq_len + 1), generator=g)
    # a learnable stream: every other token repeats its predecessor
    tok[:, 1::2] = tok[:, 0:-1:2]
    losses.append(float(t.step(tok[:, :-1].contiguous(), tok[:, 1:].contiguous())))
    if log_every and (s + 1) % log_every == 0:
      print_fn(f"step {s + 1:>4}  loss {losses[-1]:.4f}  lr {t.lr:.2e}")
  return losses


def compare(curves: Dict[str, Sequence[float]], last: int = 5) -> List[Row]:
  """First loss, mean of the last ``last`` losses and their difference, per named curve."""
  return [{"run": k, "first": float(v[0]), f"mean_last_{last}": sum(v[-last:]) / len(v[-last:]),
           "drop": float(v[0]) - sum(v[-last:]) / len(v[-last:])} for k, v in curves.items()]
