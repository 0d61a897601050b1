"""Router and MoE layer (sigmoid aux-loss-free routing or softmax, optional device-limited
routing, routed experts through RDEP, shared expert MLP).  Reference: nmoe/model.py:51-138.
"""
from __future__ import annotations

from typing import Optional

import torch
from .init import normal_, trunc_normal_
from torch import nn

from .. import ops
from ..parallel import rdep as rdep_mod
from .mlp import MLP


class Router(nn.Module):
  def __init__(self, cfg, dtype: torch.dtype = torch.bfloat16):
    super().__init__()
    self.n_experts, self.topk = cfg.n_routed_experts, cfg.n_activated_experts
    self.route_scale = float(cfg.route_scale)
    self.kind = cfg.router_type
    self.max_groups = int(cfg.route_max_devices)
    self.n_groups = int(cfg.route_n_groups)
    self.gate = nn.Parameter(torch.empty(self.n_experts, cfg.dim, dtype=dtype))
    self.register_buffer("bias", torch.zeros(self.n_experts, dtype=torch.float32))

  def init_weights(self, init_std: float = 0.02) -> None:
    trunc_normal_(self.gate, mean=0.0, std=init_std)

  def forward(self, x: torch.Tensor, loads: Optional[torch.Tensor] = None):
    logits = ops.linear(x, self.gate)
    return ops.router_topk(logits, self.bias if self.kind == "sigmoid" else None, self.topk,
                           route_scale=self.route_scale, kind=self.kind, n_groups=self.n_groups,
                           max_groups=self.max_groups, loads=loads)

  @torch.no_grad()
  def update_bias(self, loads: torch.Tensor, gamma: float) -> None:
    ops.router_bias_update_(self.bias, loads, gamma)


_SIDE_STREAMS = {}


def _side_stream(device: torch.device) -> "torch.cuda.Stream":
  s = _SIDE_STREAMS.get(device)
  if s is None:
    s = torch.cuda.Stream(device=device)
    _SIDE_STREAMS[device] = s
  return s


class MoE(nn.Module):
  """Routed experts (this rank holds ``n_local`` of them) + shared expert MLP."""

  def __init__(self, cfg, layer_id: int, *, rdep: Optional["rdep_mod.Rdep"], n_local: int,
               dtype: torch.dtype = torch.bfloat16):
    super().__init__()
    self.dim = cfg.dim
    self.inter = cfg.moe_inter_dim or cfg.inter_dim
    self.n_local, self.K = n_local, cfg.n_activated_experts
    self.rdep = rdep
    self.router = Router(cfg, dtype)
    self.W13 = nn.Parameter(torch.empty(n_local, 2 * self.inter, self.dim, dtype=dtype))
    self.W2 = nn.Parameter(torch.empty(n_local, self.dim, self.inter, dtype=dtype))
    self.shared = MLP(self.dim, cfg.n_shared_experts * self.inter, dtype) if cfg.n_shared_experts else None
    self.register_buffer("loads", torch.zeros(cfg.n_routed_experts, dtype=torch.int32), persistent=False)
    self.save_h13 = bool(getattr(cfg, "moe_save_h13", False))
    self.expert_dtype = cfg.dtype
    self._wcache = None
    # run the shared-expert MLP on a second stream next to the routed experts: its GEMMs fill the stretches in which the
    # routed path moves rows (placement, return, K-way sum) or waits for its peers.  Measured on ONE GPU, where there is
    # nobody to wait for: 411.1 / 412.3 -> 406.3 / 408.0 ms per Moonlight step; more with peers.
    ov = getattr(cfg, "moe_overlap_shared", "auto")
    self.overlap_shared = (rdep is not None) if ov == "auto" else str(ov).lower() in ("1", "true", "yes")

  def init_weights(self, init_std: float = 0.02) -> None:
    for W in (self.W13, self.W2):
      trunc_normal_(W, mean=0.0, std=init_std)
    self.router.init_weights(init_std)
    if self.shared is not None:
      self.shared.init_weights(init_std)

  def forward(self, x: torch.Tensor) -> torch.Tensor:
    X = x.reshape(-1, x.size(-1))
    gates, eid = self.router(X, self.loads)
    if X.is_cuda:
      wq = None
      if self.expert_dtype != "bf16":
        if self._wcache is None:
          from ..ops.quant import NVFP4_PROFILE, ExpertWeightCache, ExpertWeightCacheNV16
          self._wcache = ExpertWeightCacheNV16() if self.expert_dtype == NVFP4_PROFILE else ExpertWeightCache(self.expert_dtype)
        wq = self._wcache.get(self.W13, self.W2)
      if self.shared is not None and self.overlap_shared:
        cur = torch.cuda.current_stream()
        side = _side_stream(X.device)
        side.wait_stream(cur)
        with torch.cuda.stream(side):
          sh = self.shared(X)
        X.record_stream(side)
        out = self.rdep.moe(X, gates, eid, self.W13, self.W2, self.save_h13, wq)
        cur.wait_stream(side)
        sh.record_stream(cur)
        return (out + sh).view_as(x)
      out = self.rdep.moe(X, gates, eid, self.W13, self.W2, self.save_h13, wq)
    else:
      out = rdep_mod.moe_reference(X, gates, eid, self.W13, self.W2)
    if self.shared is not None:
      out = out + self.shared(X)
    return out.view_as(x)
