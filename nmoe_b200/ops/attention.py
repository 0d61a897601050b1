"""Softmax attention entry point: causal, optional sliding window, optional learned sinks, GQA.

q,k: [B,S,Hq|Hkv,Dqk]; v: [B,S,Hkv,Dv] -> [B,S,Hq,Dv].  MLA calls it with (Dqk,Dv)=(192,128).

Forward on CUDA = the tcgen05 kernel in ``csrc/attention.cu`` (head dims (192,128), (128,128),
(64,64)); it also returns the log-sum-exp.  Backward on CUDA = the two tcgen05 kernels in
``csrc/attention_bwd.cu`` (dK/dV per key block, dQ per query block), for every mask form the
forward supports.  CPU tensors run the fp32 oracle.
"""
from __future__ import annotations

import ctypes
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


class SparseMask:
  """Which keys each query may attend, on top of the causal rule: one bit per (query, key), shared by all heads.

  On CUDA the mask is a packed bit matrix ``bits`` [B, S, W] (int32 words, W = 2*ceil(S/64)) that the attention
  kernels test in their softmax stage, plus its bit transpose for the dK/dV kernel; nothing of size [B, H, S, S] is
  ever built.  On CPU it is a bool tensor [B, S, S] for the fp32 oracle.  Producers (csrc/sparse_mask.cu):

    from_topk_scores   per query, the k best-scoring keys among those at or before it (DeepSeek sparse attention)
    from_blocks        per query, every key of a list of selected key blocks (NSA selection branch)
    from_positions     one set of key positions for all queries (NSA compressed branch)
  """

  def __init__(self, B: int, S: int, bits: Optional[torch.Tensor] = None, dense: Optional[torch.Tensor] = None):
    self.B, self.S, self.bits, self.dense = B, S, bits, dense
    self._bits_t: Optional[torch.Tensor] = None

  @staticmethod
  def words(S: int) -> int:
    return 2 * ((S + 63) // 64)

  @classmethod
  def from_topk_scores(cls, scores: torch.Tensor, k: int) -> "SparseMask":
    """scores [B, S, S] fp32, row q = scores of the keys (-inf = never); entries above the diagonal are ignored."""
    B, S, _ = scores.shape
    if not scores.is_cuda:
      s = scores.float().masked_fill(torch.triu(torch.ones(S, S, dtype=torch.bool), 1), float("-inf"))
      kk = min(k, S)
      vals, idx = s.topk(kk, dim=-1)
      dense = torch.zeros(B, S, S, dtype=torch.bool)
      dense.scatter_(2, idx, vals > float("-inf"))
      return cls(B, S, dense=dense)
    scores = scores.float().contiguous()
    bits = torch.empty(B, S, cls.words(S), dtype=torch.int32, device=scores.device)
    L.check(L.lib().nmoe_mask_topk(L.ptr(scores), B, S, int(k), L.ptr(bits), L.stream()), "mask_topk")
    return cls(B, S, bits=bits)

  @classmethod
  def from_blocks(cls, blocks: torch.Tensor, block_size: int, S: int) -> "SparseMask":
    """blocks [B, S, n] integer key-block indices per query (-1 = unused slot)."""
    B = blocks.size(0)
    if not blocks.is_cuda:
      nb = (S + block_size - 1) // block_size
      onehot = torch.zeros(B, S, nb + 1, dtype=torch.bool)
      onehot.scatter_(2, blocks.long().clamp(min=-1).add(0).where(blocks >= 0, torch.full_like(blocks, nb)).long(), True)
      dense = onehot[..., :nb].repeat_interleave(block_size, dim=-1)[..., :S]
      return cls(B, S, dense=dense)
    blocks = blocks.to(torch.int32).contiguous()
    bits = torch.empty(B, S, cls.words(S), dtype=torch.int32, device=blocks.device)
    L.check(L.lib().nmoe_mask_from_blocks(L.ptr(blocks), B, S, blocks.size(2), int(block_size), L.ptr(bits), L.stream()),
            "mask_from_blocks")
    return cls(B, S, bits=bits)

  @classmethod
  def from_positions(cls, positions: torch.Tensor, B: int, S: int) -> "SparseMask":
    """positions: 1-D integer key positions that every query may attend (subject to causality)."""
    if not positions.is_cuda:
      row = torch.zeros(S, dtype=torch.bool)
      row[positions.long()[(positions >= 0) & (positions < S)]] = True
      return cls(B, S, dense=row.view(1, 1, S).expand(B, S, S))
    positions = positions.to(torch.int32).contiguous()
    bits = torch.empty(B, S, cls.words(S), dtype=torch.int32, device=positions.device)
    L.check(L.lib().nmoe_mask_positions(L.ptr(positions), positions.numel(), B, S, L.ptr(bits), L.stream()),
            "mask_positions")
    return cls(B, S, bits=bits)

  @property
  def bits_t(self) -> torch.Tensor:
    if self._bits_t is None:
      self._bits_t = torch.empty_like(self.bits)
      L.check(L.lib().nmoe_mask_transpose(L.ptr(self.bits), L.ptr(self._bits_t), self.B, self.S, L.stream()),
              "mask_transpose")
    return self._bits_t

  def to_bool(self) -> torch.Tensor:
    """[B, S, S] bool (tests and the CPU oracle)."""
    if self.dense is not None:
      return self.dense
    w = self.bits.to(torch.int64) & 0xFFFFFFFF
    sh = torch.arange(32, device=w.device, dtype=torch.int64)
    return ((w.unsqueeze(-1) >> sh) & 1).bool().view(self.B, self.S, -1)[..., :self.S]


def attention_forward(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, window: int = 0,
                      sinks: Optional[torch.Tensor] = None, need_lse: bool = True, mask: Optional[SparseMask] = None):
  """Raw kernel call (no autograd): returns (o [B,S,Hq,Dv] bf16, lse [B,Hq,S] fp32 or None)."""
  B, S, Hq, Dqk = q.shape
  Hkv, Dv = k.size(2), v.size(3)
  q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
  o = torch.empty(B, S, Hq, Dv, dtype=q.dtype, device=q.device)
  lse = torch.empty(B, Hq, S, dtype=torch.float32, device=q.device) if need_lse else None
  sk = sinks.detach().float().contiguous() if sinks is not None else None
  st = status_buffer(q.device)
  L.check(L.lib().nmoe_attn_fwd_masked(
    L.ptr(q), Hq * Dqk, Dqk, L.ptr(k), Hkv * Dqk, Dqk, 0, Dqk // 64, None, 0, 0, 0, L.ptr(v), Hkv * Dv, Dv, 0,
    L.ptr(o), L.ptr(lse), L.ptr(sk), L.ptr(mask.bits) if mask is not None else None, B, S, Hq, Hkv, Dqk, Dv,
    int(window), L.c_float(scale), L.ptr(st), L.stream()), "attn_fwd")
  return o, lse


def attention_backward(q, k, v, o, do, lse, scale: float, window: int = 0, mask: Optional[SparseMask] = None):
  """Raw backward kernels (``csrc/attention_bwd.cu``): returns (dq, dk, dv, delta).

  ``delta`` [B,Hq,S] = rowsum(o * do) is what the sink gradient needs besides ``lse``."""
  B, S, Hq, Dqk = q.shape
  Hkv, Dv = k.size(2), v.size(3)
  q, k, v, o, do = (t.contiguous() for t in (q, k, v, o, do))
  g = Hq // Hkv
  dq = torch.empty_like(q)
  dk = torch.empty(B, S, Hq, Dqk, dtype=q.dtype, device=q.device)
  dv = torch.empty(B, S, Hq, Dv, dtype=q.dtype, device=q.device)
  delta = torch.empty(B, Hq, S, dtype=torch.float32, device=q.device)
  addr = (ctypes.c_int * 11)(Hq * Dqk, Dqk, Hq * Dqk, Dqk, 0, Hq * Dqk, Dqk, 0, Hq * Dv, Dv, 0)
  st = status_buffer(q.device)
  L.check(L.lib().nmoe_attn_bwd_masked(
    L.ptr(q), Hq * Dqk, Dqk, L.ptr(k), Hkv * Dqk, Dqk, 0, Dqk // 64, None, 0, 0, 0, L.ptr(v), Hkv * Dv, Dv, 0,
    L.ptr(o), L.ptr(do), L.ptr(lse), L.ptr(delta), L.ptr(dq), L.ptr(dk), None, L.ptr(dv), addr,
    L.ptr(mask.bits) if mask is not None else None, L.ptr(mask.bits_t) if mask is not None else None,
    B, S, Hq, Hkv, Dqk, Dv, int(window), L.c_float(scale), L.ptr(st), L.stream()), "attn_bwd", 3)
  if g > 1:   # one slot per query head -> sum the group
    dk = dk.view(B, S, Hkv, g, Dqk).sum(3, dtype=torch.float32).to(q.dtype)
    dv = dv.view(B, S, Hkv, g, Dv).sum(3, dtype=torch.float32).to(q.dtype)
  return dq, dk, dv, delta


class _Attention(torch.autograd.Function):
  @staticmethod
  def forward(ctx, q, k, v, sinks, scale, window, mask=None):
    o, lse = attention_forward(q, k, v, scale, window, sinks, need_lse=True, mask=mask)
    ctx.save_for_backward(q, k, v, sinks, o, lse)
    ctx.scale, ctx.window, ctx.mask = scale, window, mask
    return o

  @staticmethod
  def backward(ctx, do):
    q, k, v, sinks, o, lse = ctx.saved_tensors
    dq, dk, dv, delta = attention_backward(q, k, v, o, do, lse, ctx.scale, ctx.window, ctx.mask)
    ds = None
    if sinks is not None:
      # the sink is one more logit with a zero value row: dsink = -sum_rows P_sink * delta
      ds = -(torch.exp(sinks.detach().float().view(1, -1, 1) - lse) * delta).sum((0, 2)).to(sinks.dtype)
    return dq, dk, dv, ds, None, None, None


class _MLAAttention(torch.autograd.Function):
  """MLA core attention reading k_nope / v straight out of the fused kv projection output and the
  shared rotary key from its own tensor: neither direction materialises K [B,S,H,192] or a
  contiguous V.  The backward writes d(k_nope) and dv into one [B,S,H,nope+vdim] buffer (the
  gradient of the kv projection output) and the per-head rotary-key gradients into a small
  buffer that is summed over heads."""

  @staticmethod
  def forward(ctx, q, kv, k_pe, scale, nope, vdim):
    B, S, H, Dqk = q.shape
    rope = Dqk - nope
    q, kv, k_pe = q.contiguous(), kv.contiguous(), k_pe.contiguous()
    o = torch.empty(B, S, H, vdim, dtype=q.dtype, device=q.device)
    lse = torch.empty(B, H, S, dtype=torch.float32, device=q.device)
    st = status_buffer(q.device)
    row_kv = H * (nope + vdim)
    L.check(L.lib().nmoe_attn_fwd_ex(
      L.ptr(q), H * Dqk, Dqk, L.ptr(kv), row_kv, nope + vdim, 0, nope // 64, L.ptr(k_pe), rope, 0, 0,
      L.ptr(kv), row_kv, nope + vdim, nope, L.ptr(o), L.ptr(lse), None, B, S, H, H, Dqk, vdim, 0, L.c_float(scale),
      L.ptr(st), L.stream()), "attn_fwd(mla)")
    ctx.save_for_backward(q, kv, k_pe, o, lse)
    ctx.args = (scale, nope, vdim)
    return o

  @staticmethod
  def backward(ctx, do):
    q, kv, k_pe, o, lse = ctx.saved_tensors
    scale, nope, vdim = ctx.args
    B, S, H, Dqk = q.shape
    rope = Dqk - nope
    do = do.contiguous()
    dq = torch.empty_like(q)
    dkv = torch.empty_like(kv)
    dpe_h = torch.empty(B, S, H, rope, dtype=q.dtype, device=q.device)
    delta = torch.empty(B, H, S, dtype=torch.float32, device=q.device)
    row_kv = H * (nope + vdim)
    addr = (ctypes.c_int * 11)(H * Dqk, Dqk, row_kv, nope + vdim, 0, H * rope, rope, 0, row_kv, nope + vdim, nope)
    st = status_buffer(q.device)
    L.check(L.lib().nmoe_attn_bwd_ex(
      L.ptr(q), H * Dqk, Dqk, L.ptr(kv), row_kv, nope + vdim, 0, nope // 64, L.ptr(k_pe), rope, 0, 0,
      L.ptr(kv), row_kv, nope + vdim, nope, L.ptr(o), L.ptr(do), L.ptr(lse), L.ptr(delta), L.ptr(dq), L.ptr(dkv),
      L.ptr(dpe_h), L.ptr(dkv), addr, B, S, H, H, Dqk, vdim, 0, L.c_float(scale), L.ptr(st), L.stream()),
      "attn_bwd(mla)", 3)
    dpe = dpe_h.sum(2, keepdim=True, dtype=torch.float32).to(q.dtype)
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


def _masked_oracle(q, k, v, scale, window, sinks, mask: SparseMask):
  from ..models.attention.common import masked_attention
  S = q.size(1)
  i = torch.arange(S, device=q.device).unsqueeze(-1)
  j = torch.arange(S, device=q.device).unsqueeze(0)
  allowed = mask.to_bool().to(q.device) & (j <= i)
  if window > 0:
    allowed = allowed & (j > i - window)
  return masked_attention(q, k, v, allowed.unsqueeze(1), scale, sinks)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, *, causal: bool = True,
              window: int = 0, sinks: Optional[torch.Tensor] = None, mask: Optional[SparseMask] = None) -> torch.Tensor:
  """``mask`` restricts every query to a subset of the keys it could causally see (see SparseMask)."""
  if not q.is_cuda:
    if mask is not None:
      return _masked_oracle(q, k, v, scale, window, sinks, mask)
    return R.attention(q, k, v, scale, causal=causal, window=window, sinks=sinks)
  assert causal, "only causal attention is used by this framework"
  if (q.size(-1), v.size(-1)) in _KERNEL_DIMS and q.dtype == torch.bfloat16:
    return _Attention.apply(q, k, v, sinks, scale, int(window), mask)
  if mask is not None:
    return _masked_oracle(q, k, v, scale, window, sinks, mask)
  if window > 0 or sinks is not None:
    return _banded_eager(q, k, v, scale, window, sinks)
  Hq, Hkv = q.size(2), k.size(2)
  o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True,
                                     scale=scale, enable_gqa=(Hq != Hkv))
  return o.transpose(1, 2)
