"""Softmax attention entry point: causal, optional sliding window, optional learned sinks, GQA.

q,k: [B,S,Hq|Hkv,Dqk]; v: [B,S,Hkv,Dv] -> [B,S,Hq,Dv].  MLA calls it with (Dqk,Dv)=(192,128).

Forward on CUDA = the tcgen05 kernel in ``csrc/attention.cu`` (head dims (192,128), (128,128),
(64,64)); it also returns the log-sum-exp.  Backward: full-causal attention without sinks goes
through the cuDNN fused backward (recomputed from q,k,v); windowed / sink attention differentiates
a query-block-tiled eager statement.  CPU tensors run the fp32 oracle.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F

from ..ref import ops as R
from . import _lib as L
from .tc_gemm import status_buffer

_KERNEL_DIMS = {(192, 128), (128, 128), (64, 64)}


def _banded_eager(q, k, v, scale, window, sinks):
  """Query-block tiled eager attention (library GEMMs), differentiable.

  Each block of ``bq`` queries only sees keys in [start - window + 1, end], so the cost is
  O(S * (bq + window)) instead of O(S^2) when a window is set.
  """
  B, S, Hq, Dqk = q.shape
  Hkv = k.size(2)
  if Hkv != Hq:
    k = k.repeat_interleave(Hq // Hkv, dim=2)
    v = v.repeat_interleave(Hq // Hkv, dim=2)
  bq = 512
  outs = []
  for s0 in range(0, S, bq):
    s1 = min(S, s0 + bq)
    k0 = max(0, s0 - window + 1) if window > 0 else 0
    qs = q[:, s0:s1].transpose(1, 2).float()
    ks = k[:, k0:s1].transpose(1, 2).float()
    vs = v[:, k0:s1].transpose(1, 2).float()
    s = torch.matmul(qs, ks.transpose(-1, -2)) * scale
    i = torch.arange(s0, s1, device=q.device).unsqueeze(-1)
    j = torch.arange(k0, s1, device=q.device).unsqueeze(0)
    mask = j <= i
    if window > 0:
      mask &= j > i - window
    s = s.masked_fill(~mask, float("-inf"))
    if sinks is not None:
      sk = sinks.float().view(1, Hq, 1, 1).expand(B, Hq, s1 - s0, 1)
      p = torch.softmax(torch.cat((s, sk), dim=-1), dim=-1)[..., :-1]
    else:
      p = torch.softmax(s, dim=-1)
    outs.append(torch.matmul(p, vs).transpose(1, 2))
  return torch.cat(outs, dim=1).to(q.dtype)


def attention_forward(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, window: int = 0,
                      sinks: Optional[torch.Tensor] = None, need_lse: bool = True):
  """Raw kernel call (no autograd): returns (o [B,S,Hq,Dv] bf16, lse [B,Hq,S] fp32 or None)."""
  B, S, Hq, Dqk = q.shape
  Hkv, Dv = k.size(2), v.size(3)
  q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
  o = torch.empty(B, S, Hq, Dv, dtype=q.dtype, device=q.device)
  lse = torch.empty(B, Hq, S, dtype=torch.float32, device=q.device) if need_lse else None
  sk = sinks.detach().float().contiguous() if sinks is not None else None
  st = status_buffer(q.device)
  L.check(L.lib().nmoe_attn_fwd(L.ptr(q), L.ptr(k), L.ptr(v), L.ptr(o), L.ptr(lse), L.ptr(sk), B, S, Hq, Hkv, Dqk, Dv,
                                int(window), L.c_float(scale), L.ptr(st), L.stream()), "attn_fwd")
  return o, lse


class _Attention(torch.autograd.Function):
  @staticmethod
  def forward(ctx, q, k, v, sinks, scale, window):
    o, lse = attention_forward(q, k, v, scale, window, sinks, need_lse=False)
    ctx.save_for_backward(q, k, v, sinks)
    ctx.scale, ctx.window = scale, window
    return o

  @staticmethod
  def backward(ctx, do):
    q, k, v, sinks = ctx.saved_tensors
    scale, window = ctx.scale, ctx.window
    with torch.enable_grad():
      qd, kd, vd = (t.detach().requires_grad_() for t in (q, k, v))
      sd = sinks.detach().requires_grad_() if sinks is not None else None
      if window == 0 and sinks is None:
        Hq, Hkv = q.size(2), k.size(2)
        o2 = F.scaled_dot_product_attention(qd.transpose(1, 2), kd.transpose(1, 2), vd.transpose(1, 2), is_causal=True,
                                            scale=scale, enable_gqa=(Hq != Hkv)).transpose(1, 2)
      else:
        o2 = _banded_eager(qd, kd, vd, scale, window, sd)
      ins = (qd, kd, vd) + ((sd,) if sd is not None else ())
      grads = torch.autograd.grad(o2, ins, do)
    dq, dk, dv = grads[:3]
    ds = grads[3].to(sinks.dtype) if sd is not None else None
    return dq, dk, dv, ds, None, None


class _MLAAttention(torch.autograd.Function):
  """MLA core attention reading k_nope / v straight out of the fused kv projection output and the
  shared rotary key from its own tensor: the forward never materialises K [B,S,H,192] or a
  contiguous V.  The backward assembles them once and uses the library fused backward."""

  @staticmethod
  def forward(ctx, q, kv, k_pe, scale, nope, vdim):
    B, S, H, Dqk = q.shape
    rope = Dqk - nope
    q, kv, k_pe = q.contiguous(), kv.contiguous(), k_pe.contiguous()
    o = torch.empty(B, S, H, vdim, dtype=q.dtype, device=q.device)
    st = status_buffer(q.device)
    row_kv = H * (nope + vdim)
    L.check(L.lib().nmoe_attn_fwd_ex(
      L.ptr(q), H * Dqk, Dqk, L.ptr(kv), row_kv, nope + vdim, 0, nope // 64, L.ptr(k_pe), rope, 0, 0,
      L.ptr(kv), row_kv, nope + vdim, nope, L.ptr(o), None, None, B, S, H, H, Dqk, vdim, 0, L.c_float(scale),
      L.ptr(st), L.stream()), "attn_fwd(mla)")
    ctx.save_for_backward(q, kv, k_pe)
    ctx.args = (scale, nope, vdim)
    return o

  @staticmethod
  def backward(ctx, do):
    q, kv, k_pe = ctx.saved_tensors
    scale, nope, vdim = ctx.args
    B, S, H, _ = q.shape
    with torch.enable_grad():
      qd, kvd, ped = (t.detach().requires_grad_() for t in (q, kv, k_pe))
      k = torch.cat((kvd[..., :nope], ped.expand(B, S, H, ped.size(-1))), dim=-1)
      v = kvd[..., nope:]
      o2 = F.scaled_dot_product_attention(qd.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True,
                                          scale=scale).transpose(1, 2)
      dq, dkv, dpe = torch.autograd.grad(o2, (qd, kvd, ped), do)
    return dq, dkv, dpe, None, None, None


def mla_attention(q: torch.Tensor, kv: torch.Tensor, k_pe: torch.Tensor, scale: float, nope: int, vdim: int) -> torch.Tensor:
  """q [B,S,H,nope+rope] (rotary applied), kv [B,S,H,nope+vdim] (k_nope | v per head), k_pe [B,S,1,rope]
  (rotary applied, shared by all heads) -> [B,S,H,vdim], full causal."""
  rope = q.size(-1) - nope
  if q.is_cuda and q.dtype == torch.bfloat16 and (q.size(-1), vdim) in _KERNEL_DIMS and nope % 64 == 0 and rope % 64 == 0:
    return _MLAAttention.apply(q, kv, k_pe, scale, nope, vdim)
  B, S, H, _ = q.shape
  k = torch.cat((kv[..., :nope], k_pe.expand(B, S, H, rope)), dim=-1)
  return attention(q, k, kv[..., nope:].contiguous(), scale)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, *, causal: bool = True,
              window: int = 0, sinks: Optional[torch.Tensor] = None) -> torch.Tensor:
  if not q.is_cuda:
    return R.attention(q, k, v, scale, causal=causal, window=window, sinks=sinks)
  assert causal, "only causal attention is used by this framework"
  if (q.size(-1), v.size(-1)) in _KERNEL_DIMS and q.dtype == torch.bfloat16:
    return _Attention.apply(q, k, v, sinks, scale, int(window))
  if window > 0 or sinks is not None:
    return _banded_eager(q, k, v, scale, window, sinks)
  Hq, Hkv = q.size(2), k.size(2)
  o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True,
                                     scale=scale, enable_gqa=(Hq != Hkv))
  return o.transpose(1, 2)
