"""ZeRO-2 for the replicated (non-expert) parameters.

Each parameter group is flattened once into one bf16 parameter buffer and one bf16 gradient
buffer; parameters and their ``.grad`` become views, so there is no per-step packing copy
(the reference packs with a Python double loop, nmoe/zero2.py:233-253).  Rank r owns shard r
of each buffer and keeps AdamW moments only for it.

Three step implementations with identical math (bf16 moments, fp32 arithmetic, decay first):
  world == 1   one flat AdamW kernel per group
  "nccl"       reduce_scatter_tensor(AVG) -> flat AdamW on the shard -> all_gather_into_tensor
               (the library baseline, nmoe/zero2.py:221-279)
  "fused"      one kernel per group that reads the peers' gradient shards over NVLink, applies
               AdamW and stores the new parameters into every peer's buffer (csrc/zero2.cu)
State-dict keys follow the reference: ``shard_{rank}_{group}_{dtype}`` -> {step, exp_avg, exp_avg_sq}.
"""
from __future__ import annotations

import ctypes
import os
from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from .. import ops
from ..config import Config
from ..ops import _lib as L
from ..ops import tc_gemm as G
from ..metrics import span
from .peer import PeerSlab

_ALIGN = 256   # elements; keeps every shard 16-byte aligned and vectorisable


class _FlatGroup:
  def __init__(self, gi: int, group: dict, world: int, rank: int, device: torch.device, dtype: torch.dtype,
               slab: Optional[PeerSlab], slab_prefix: str):
    self.gi, self.name = gi, group["name"]
    self.lr, self.wd = float(group["lr"]), float(group["weight_decay"])
    self.params: List[torch.nn.Parameter] = list(group["params"])
    self.dtype = dtype
    n = sum(p.numel() for p in self.params)
    unit = world * _ALIGN
    self.total = ((n + unit - 1) // unit) * unit
    self.shard = self.total // world
    self.rank, self.world = rank, world
    if slab is not None:
      self.flat_param = slab.local(slab_prefix + "p", dtype, (self.total,))
      self.flat_grad = slab.local(slab_prefix + "g", dtype, (self.total,))
    else:
      self.flat_param = torch.zeros(self.total, dtype=dtype, device=device)
      self.flat_grad = torch.zeros(self.total, dtype=dtype, device=device)
    off = 0
    for p in self.params:
      k = p.numel()
      self.flat_param[off:off + k].copy_(p.data.reshape(-1))
      p.data = self.flat_param[off:off + k].view_as(p.data)
      p.grad = self.flat_grad[off:off + k].view_as(p.data)
      off += k
    self.exp_avg = torch.zeros(self.shard, dtype=dtype, device=device)
    self.exp_avg_sq = torch.zeros(self.shard, dtype=dtype, device=device)
    self.step = 0

  def relink_grads(self) -> None:
    """Re-point ``.grad`` at the flat buffer (someone may have set it to None)."""
    off = 0
    for p in self.params:
      k = p.numel()
      if p.grad is None or p.grad.data_ptr() != self.flat_grad.data_ptr() + off * self.flat_grad.element_size():
        p.grad = self.flat_grad[off:off + k].view_as(p.data)
      off += k


class Zero2:
  def __init__(self, groups: List[dict], cfg: Config, *, group: Optional[dist.ProcessGroup] = None):
    self.cfg = cfg
    self.pg = group
    self.world = dist.get_world_size(group) if dist.is_initialized() else 1
    self.rank = dist.get_rank(group) if dist.is_initialized() else 0
    self.betas = (cfg.adam_beta1, cfg.adam_beta2)
    self.eps = cfg.adam_eps
    self.gradnorm_sq: Optional[torch.Tensor] = None
    self.groups: List[_FlatGroup] = []
    live = [g for g in groups if g["params"]]
    if not live:
      self.impl = "none"
      return
    p0 = live[0]["params"][0]
    self.device, dtype = p0.device, p0.dtype
    impl = os.environ.get("NMOE_ZERO2_IMPL", cfg.zero2_impl)
    on_gpu = self.device.type == "cuda" and dtype == torch.bfloat16
    if self.world == 1:
      impl = "single"
    elif impl == "auto":
      impl = "fused" if on_gpu else "nccl"
    self.impl = impl
    slab = None
    if impl == "fused":
      unit = self.world * _ALIGN
      regions = []
      for gi, g in enumerate(live):
        n = sum(p.numel() for p in g["params"])
        tot = ((n + unit - 1) // unit) * unit
        regions += [(f"g{gi}p", tot * 2), (f"g{gi}g", tot * 2)]
      regions += [("ready", 64), ("done", 64)]
      slab = PeerSlab(regions, group)
      self.done_counter = torch.zeros(1, dtype=torch.int32, device=self.device)
    self.slab = slab
    self.epoch = 0
    for gi, g in enumerate(live):
      self.groups.append(_FlatGroup(gi, g, self.world, self.rank, self.device, dtype, slab, f"g{gi}"))

  # ------------------------------------------------------------------ per-step API
  def set_lrs(self, lrs: Dict[str, float]) -> None:
    for g in self.groups:
      g.lr = lrs["router"] if g.name == "router" else lrs["dense"]

  def zero_grad(self) -> None:
    for g in self.groups:
      g.flat_grad.zero_()
      g.relink_grads()

  @torch.no_grad()
  def step(self) -> None:
    for g in self.groups:
      g.step += 1
      kw = dict(lr=g.lr, beta1=self.betas[0], beta2=self.betas[1], eps=self.eps, weight_decay=g.wd, step=g.step)
      if self.impl == "single":
        if self.gradnorm_sq is not None:
          ops.sumsq(g.flat_grad, self.gradnorm_sq)
        ops.adamw_flat_(g.flat_param, g.flat_grad, g.exp_avg, g.exp_avg_sq, **kw)
      elif self.impl == "nccl":
        lo = self.rank * g.shard
        gshard = torch.empty(g.shard, dtype=g.flat_grad.dtype, device=self.device)
        if g.flat_grad.is_cuda:
          with span("time_ms/zero2_reduce_scatter"):
            dist.reduce_scatter_tensor(gshard, g.flat_grad, op=dist.ReduceOp.AVG, group=self.pg)
        else:  # gloo has no reduce_scatter: all_reduce then slice (CPU tests only)
          full = g.flat_grad.float()
          dist.all_reduce(full, group=self.pg)
          gshard = (full[lo:lo + g.shard] / self.world).to(g.flat_grad.dtype)
        if self.gradnorm_sq is not None:
          ops.sumsq(gshard, self.gradnorm_sq)
        pshard = g.flat_param[lo:lo + g.shard]
        ops.adamw_flat_(pshard, gshard, g.exp_avg, g.exp_avg_sq, **kw)
        if g.flat_param.is_cuda:
          with span("time_ms/zero2_all_gather"):
            dist.all_gather_into_tensor(g.flat_param, pshard.clone(), group=self.pg)
        else:
          parts = [torch.empty_like(pshard) for _ in range(self.world)]
          dist.all_gather(parts, pshard.clone(), group=self.pg)
          g.flat_param.copy_(torch.cat(parts))
      elif self.impl == "fused":
        self.epoch += 1
        st = G.status_buffer(self.device)
        _t = span("time_ms/zero2_fused")      # reduce-scatter + AdamW + all-gather in one kernel, plus the done wait
        _t.__enter__()
        L.check(L.lib().nmoe_zero2_fused(
          self.rank, self.world, L.c_ll(g.shard), self.slab.ptrs(f"g{g.gi}g"), self.slab.ptrs(f"g{g.gi}p"),
          self.slab.ptrs("ready"), self.slab.ptrs("done"), L.ptr(g.exp_avg), L.ptr(g.exp_avg_sq),
          L.c_float(g.lr), L.c_float(self.betas[0]), L.c_float(self.betas[1]), L.c_float(self.eps),
          L.c_float(g.wd), g.step, L.c_float(1.0 / self.world), ctypes.c_uint(self.epoch), ctypes.c_uint(0),
          L.ptr(self.done_counter), L.ptr(self.gradnorm_sq), L.ptr(st), L.stream()), "zero2_fused")
        L.check(L.lib().nmoe_rdep_wait(ctypes.c_void_p(self.slab.local_ptr("done")), self.world,
                                       ctypes.c_uint(self.epoch), ctypes.c_uint(0), L.ptr(st), 501, L.stream()),
                "zero2_wait")
        _t.__exit__(None, None, None)
      else:
        raise ValueError(f"unknown zero2 implementation {self.impl!r}")

  # ------------------------------------------------------------------ checkpoint state
  def state_dict(self) -> dict:
    out = {}
    for g in self.groups:
      key = f"shard_{self.rank}_{g.gi}_{str(g.dtype).replace('torch.', '')}"
      out[key] = {"step": g.step, "exp_avg": g.exp_avg, "exp_avg_sq": g.exp_avg_sq}
    return out

  def load_state_dict(self, sd: dict) -> None:
    for g in self.groups:
      key = f"shard_{self.rank}_{g.gi}_{str(g.dtype).replace('torch.', '')}"
      if key not in sd:
        raise KeyError(f"ZeRO-2 state has no entry {key} (was the checkpoint written with another world size?)")
      g.step = int(sd[key]["step"])
      g.exp_avg.copy_(sd[key]["exp_avg"])
      g.exp_avg_sq.copy_(sd[key]["exp_avg_sq"])
