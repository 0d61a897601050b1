"""Compressed-branch attention of Native Sparse Attention on its own kernels (csrc/nsa.cu).

``cmp_attention(q, kc, vc, T-related sizes)`` returns the branch output and the selection-block scores:

    s[t, c] = scale <q_t, kc_c>   for the compressed tokens whose block has ended by t  (c * stride + len - 1 <= t)
    p       = exp(s - max(0, max s)) / max(sum, 1e-6)
    out_t   = sum_c p[t, c] vc_c
    score[t, n] = sum of p[t, c] over the compressed tokens whose centre lies in selection block n

The scores feed a top-k and carry no gradient; ``out`` is differentiable in q, kc and vc (two backward kernels, no
atomics).  CPU tensors and unsupported head sizes run ``cmp_attention_reference``, which is also the tests' oracle.
Reference: nmoe/triton/nsa.py:27-317.
"""
from __future__ import annotations

from typing import Tuple

import torch

from . import _lib as L


def cmp_attention_reference(q, kc, vc, *, cmp_len: int, cmp_stride: int, slc_block: int, scale: float
                            ) -> Tuple[torch.Tensor, torch.Tensor]:
  """q [B,T,KV,D]; kc, vc [B,Tc,KV,D] -> (out [B,T,KV,D] in q's dtype, scores [B,T,KV,Ns] fp32)."""
  B, T, KV, D = q.shape
  Tc, Ns = kc.size(1), T // slc_block
  if Tc == 0 or Ns == 0:
    return q.new_zeros(B, T, KV, D), torch.zeros(B, T, KV, max(Ns, 1), dtype=torch.float32, device=q.device)
  s = torch.einsum("bthd,bchd->bhtc", q.float(), kc.float()) * scale
  t = torch.arange(T, device=q.device).unsqueeze(1)
  ends = torch.arange(Tc, device=q.device).unsqueeze(0) * cmp_stride + cmp_len - 1
  s = s.masked_fill((ends > t).view(1, 1, T, Tc), -1e6)
  p = torch.exp(s - s.amax(-1, keepdim=True).clamp(min=0))
  p = p / p.sum(-1, keepdim=True).clamp(min=1e-6)
  out = torch.einsum("bhtc,bchd->bthd", p, vc.float()).to(q.dtype)
  centers = torch.arange(Tc, device=q.device) * cmp_stride + cmp_len // 2
  scatter = torch.zeros(Tc, Ns, device=q.device)
  scatter[torch.arange(Tc, device=q.device), (centers // slc_block).clamp(max=Ns - 1)] = 1.0
  return out, torch.einsum("bhtc,cn->bthn", p, scatter)


def kernel_ok(q: torch.Tensor, kc: torch.Tensor, slc_block: int) -> bool:
  T = q.size(1)
  return q.is_cuda and q.dtype == torch.bfloat16 and q.size(-1) in (64, 128) and kc.size(1) > 0 \
      and 1 <= T // slc_block <= 256


class _CmpAttention(torch.autograd.Function):
  @staticmethod
  def forward(ctx, q, kc, vc, cmp_len, cmp_stride, slc_block, scale):
    B, T, KV, D = q.shape
    Tc, Ns = kc.size(1), T // slc_block
    q, kc, vc = q.contiguous(), kc.contiguous(), vc.contiguous()
    out = torch.empty_like(q)
    scores = torch.empty(B, T, KV, Ns, dtype=torch.float32, device=q.device)
    stats = torch.empty(B, KV, T, 2, dtype=torch.float32, device=q.device)
    L.check(L.lib().nmoe_nsa_cmp_fwd(L.ptr(q), L.ptr(kc), L.ptr(vc), L.ptr(out), L.ptr(scores), L.ptr(stats), B, T, KV, Tc,
                                     Ns, D, cmp_len, cmp_stride, slc_block, L.c_float(scale), L.stream()), "nsa_cmp_fwd")
    ctx.save_for_backward(q, kc, vc, out, stats)
    ctx.cfg = (cmp_len, cmp_stride, scale)
    ctx.mark_non_differentiable(scores)
    return out, scores

  @staticmethod
  def backward(ctx, dout, _dscores):
    q, kc, vc, out, stats = ctx.saved_tensors
    cmp_len, cmp_stride, scale = ctx.cfg
    B, T, KV, D = q.shape
    Tc = kc.size(1)
    dout = dout.contiguous()
    dq = torch.empty_like(q)
    dkc = torch.empty(B, Tc, KV, D, dtype=torch.float32, device=q.device)
    dvc = torch.empty_like(dkc)
    delta = torch.empty(B, KV, T, dtype=torch.float32, device=q.device)
    L.check(L.lib().nmoe_nsa_cmp_bwd(L.ptr(q), L.ptr(kc), L.ptr(vc), L.ptr(out), L.ptr(dout), L.ptr(stats), L.ptr(dq),
                                     L.ptr(dkc), L.ptr(dvc), L.ptr(delta), B, T, KV, Tc, D, cmp_len, cmp_stride,
                                     L.c_float(scale), L.stream()), "nsa_cmp_bwd", 2)
    return dq, dkc.to(kc.dtype), dvc.to(vc.dtype), None, None, None, None


def cmp_attention(q, kc, vc, *, cmp_len: int, cmp_stride: int, slc_block: int, scale: float):
  if kernel_ok(q, kc, slc_block):
    return _CmpAttention.apply(q, kc.to(q.dtype), vc.to(q.dtype), int(cmp_len), int(cmp_stride), int(slc_block), float(scale))
  return cmp_attention_reference(q, kc, vc, cmp_len=cmp_len, cmp_stride=cmp_stride, slc_block=slc_block, scale=scale)
