"""Router top-k op (``csrc/router.cu``) with autograd through the selected weights."""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from ..ref import ops as R
from . import _lib as L

_KIND = {"sigmoid": 0, "softmax": 1}


class _RouterTopK(torch.autograd.Function):
  @staticmethod
  def forward(ctx, logits, bias, topk, route_scale, kind, n_groups, max_groups, loads):
    T, E = logits.shape
    lg = logits.contiguous()
    w = torch.empty(T, topk, dtype=torch.float32, device=lg.device)
    idx = torch.empty(T, topk, dtype=torch.int32, device=lg.device)
    L.check(L.lib().nmoe_router_fwd(L.ptr(lg), int(lg.dtype == torch.float32), L.ptr(bias), T, E, topk,
                                    L.c_float(route_scale), _KIND[kind], n_groups, max_groups, L.ptr(w), L.ptr(idx),
                                    L.ptr(loads), L.stream()), "router_fwd")
    ctx.save_for_backward(lg, idx)
    ctx.args = (topk, route_scale, kind)
    ctx.mark_non_differentiable(idx)
    return w, idx

  @staticmethod
  def backward(ctx, dw, _didx):
    lg, idx = ctx.saved_tensors
    topk, route_scale, kind = ctx.args
    T, E = lg.shape
    dl = torch.empty_like(lg)
    L.check(L.lib().nmoe_router_bwd(L.ptr(lg), int(lg.dtype == torch.float32), L.ptr(idx),
                                    L.ptr(dw.float().contiguous()), T, E, topk, L.c_float(route_scale), _KIND[kind],
                                    L.ptr(dl), L.stream()), "router_bwd")
    return dl, None, None, None, None, None, None, None


def router_topk(logits: torch.Tensor, bias: Optional[torch.Tensor], topk: int, *, route_scale: float = 1.0,
                kind: str = "sigmoid", n_groups: int = 0, max_groups: int = 0,
                loads: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
  """Returns (weights fp32 [T,K], expert ids [T,K]); ``loads`` (int32 [E]) is incremented per selection."""
  if logits.is_cuda:
    return _RouterTopK.apply(logits, bias, topk, route_scale, kind, n_groups, max_groups, loads)
  w, idx = R.router(logits, bias, topk, route_scale=route_scale, kind=kind, n_groups=n_groups, max_groups=max_groups)
  if loads is not None:
    loads += torch.bincount(idx.reshape(-1), minlength=logits.size(-1)).to(loads.dtype)
  return w, idx


def router_bias_update_(bias: torch.Tensor, loads: torch.Tensor, gamma: float) -> None:
  """bias -= gamma * (s - mean s), s = sign(load/sum(load) - 1/E), clamped to +-16 (nmoe/model.py:72-77)."""
  E = bias.numel()
  if bias.is_cuda:
    L.check(L.lib().nmoe_router_bias_update(L.ptr(bias), L.ptr(loads.float().contiguous()), E, L.c_float(gamma),
                                            L.stream()), "router_bias_update")
    return
  frac = loads.float() / loads.float().sum().clamp_min(1.0)
  s = torch.sign(frac - 1.0 / E)
  bias.sub_(gamma * (s - s.mean())).clamp_(-16.0, 16.0)
