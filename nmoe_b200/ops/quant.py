"""Block-scaled quantisation ops and the MXFP8 tensor-core GEMM (``csrc/quant.cu``, ``csrc/gemm_mx.cu``).

MXFP8 = E4M3 values + one E8M0 (power-of-two) scale per 32 elements along K; scales live in the
128x4 atom layout that block-scaled ``tcgen05.mma`` consumes.  CPU tensors use the bit-exact
emulation in ``nmoe_b200.ref.quant``.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from ..ref import quant as RQ
from . import _lib as L
from .tc_gemm import status_buffer


def sf_bytes(M: int, K: int) -> int:
  return ((M + 127) // 128) * (((K // 32) + 3) // 4) * 512


def quant_mxfp8(x: torch.Tensor, n_tiles: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
  """x [M,K] bf16 -> (q uint8 [M,K] holding e4m3 bytes, sf uint8 flat buffer in atom layout)."""
  M, K = x.shape
  if not x.is_cuda:
    q, sf = RQ.quant_mxfp8(x.float())
    Mp = (M + 127) // 128 * 128
    sfp = torch.full((Mp, ((K // 32) + 3) // 4 * 4), 127, dtype=torch.uint8)
    sfp[:M, :K // 32] = sf
    return q.view(torch.uint8), RQ.sf_to_mma_layout(sfp)
  q = torch.empty(M, K, dtype=torch.uint8, device=x.device)
  sf = torch.full((sf_bytes(M, K),), 127, dtype=torch.uint8, device=x.device)
  L.check(L.lib().nmoe_quant_mxfp8(L.ptr(x.contiguous()), L.ptr(q), L.ptr(sf), L.c_ll(M), K, L.ptr(n_tiles), L.stream()),
          "quant_mxfp8")
  return q, sf


def dequant_mxfp8(q: torch.Tensor, sf: torch.Tensor) -> torch.Tensor:
  M, K = q.shape
  if not q.is_cuda:
    Mp = (M + 127) // 128 * 128
    s = RQ.sf_from_mma_layout(sf, Mp, ((K // 32) + 3) // 4 * 4)[:M, :K // 32]
    return RQ.dequant_mxfp8(q.view(torch.float8_e4m3fn), s).to(torch.bfloat16)
  out = torch.empty(M, K, dtype=torch.bfloat16, device=q.device)
  L.check(L.lib().nmoe_dequant_mxfp8(L.ptr(q), L.ptr(sf), L.ptr(out), L.c_ll(M), K, L.stream()), "dequant_mxfp8")
  return out


def swiglu_quant_mxfp8(h13: torch.Tensor, n_tiles: Optional[torch.Tensor] = None):
  """h13 [M,2F] (gate even / up odd) -> quantised silu(gate)*up: (q [M,F], sf atoms)."""
  M, F2 = h13.shape
  F = F2 // 2
  q = torch.empty(M, F, dtype=torch.uint8, device=h13.device)
  sf = torch.empty(sf_bytes(M, F), dtype=torch.uint8, device=h13.device)
  L.check(L.lib().nmoe_swiglu_quant_mxfp8(L.ptr(h13), L.ptr(q), L.ptr(sf), L.c_ll(M), F, L.ptr(n_tiles), L.stream()),
          "swiglu_quant_mxfp8")
  return q, sf


def quant_mxfp4(x: torch.Tensor):
  """x [M,K] bf16 -> (packed uint8 [M,K/2] E2M1 nibbles, sf atoms with E8M0 per 32)."""
  M, K = x.shape
  if not x.is_cuda:
    q, sf = RQ.quant_mxfp4(x.float())
    Mp = (M + 127) // 128 * 128
    sfp = torch.full((Mp, ((K // 32) + 3) // 4 * 4), 127, dtype=torch.uint8)
    sfp[:M, :K // 32] = sf
    return q, RQ.sf_to_mma_layout(sfp)
  q = torch.empty(M, K // 2, dtype=torch.uint8, device=x.device)
  sf = torch.full((sf_bytes(M, K),), 127, dtype=torch.uint8, device=x.device)
  L.check(L.lib().nmoe_quant_mxfp4(L.ptr(x.contiguous()), L.ptr(q), L.ptr(sf), L.c_ll(M), K, L.stream()), "quant_mxfp4")
  return q, sf


def gemm_mxfp8(aq: torch.Tensor, asf: torch.Tensor, bq: torch.Tensor, bsf: torch.Tensor, *,
               out: Optional[torch.Tensor] = None, bn: int = 0) -> torch.Tensor:
  """C[M,N] bf16 = dequant(A)[M,K] @ dequant(B)[N,K]^T on the block-scaled tensor-core path."""
  M, K = aq.shape
  N = bq.size(0)
  if out is None:
    out = torch.empty(M, N, dtype=torch.bfloat16, device=aq.device)
  st = status_buffer(aq.device)
  L.check(L.lib().nmoe_gemm_mxfp8(L.ptr(aq), L.ptr(asf), L.ptr(bq), L.ptr(bsf), L.ptr(out), M, N, K,
                                  L.c_ll(out.stride(0)), 0, 1, None, None, L.c_ll(M), L.c_ll(N), bn, L.ptr(st), None,
                                  None, 0, 0, L.stream()), "gemm_mxfp8")
  return out


def gemm_mxfp4(aq: torch.Tensor, asf: torch.Tensor, bq: torch.Tensor, bsf: torch.Tensor, *,
               out: Optional[torch.Tensor] = None, bn: int = 0) -> torch.Tensor:
  """C[M,N] bf16 = dequant(A) @ dequant(B)^T for MXFP4 operands (packed [M,K/2] / [N,K/2] bytes,
  E8M0 scale atoms) on ``kind::mxf4nvf4.block_scale``; K % 256 == 0."""
  M, K = aq.size(0), aq.size(1) * 2
  N = bq.size(0)
  if out is None:
    out = torch.empty(M, N, dtype=torch.bfloat16, device=aq.device)
  st = status_buffer(aq.device)
  L.check(L.lib().nmoe_gemm_mxfp4(L.ptr(aq), L.ptr(asf), L.ptr(bq), L.ptr(bsf), L.ptr(out), M, N, K,
                                  L.c_ll(out.stride(0)), 0, 1, None, None, L.c_ll(M), L.c_ll(N), bn, L.ptr(st), None,
                                  None, 0, 0, L.stream()), "gemm_mxfp4")
  return out


def grouped_gemm_mxfp4(aq: torch.Tensor, asf: torch.Tensor, bq: torch.Tensor, bsf: torch.Tensor,
                       tile_expert: torch.Tensor, n_m_tiles: torch.Tensor, *, out: Optional[torch.Tensor] = None,
                       bn: int = 0, push: Optional[dict] = None) -> Optional[torch.Tensor]:
  """Grouped form: rows of aq [Mcap,K/2] are 128-aligned expert segments; bq [E,N,K/2]."""
  Mcap, K = aq.size(0), aq.size(1) * 2
  E, N = bq.size(0), bq.size(1)
  st = status_buffer(aq.device)
  if push is not None:
    L.check(L.lib().nmoe_gemm_mxfp4(L.ptr(aq), L.ptr(asf), L.ptr(bq), L.ptr(bsf), None, Mcap, N, K, L.c_ll(N), 1, E,
                                    L.ptr(tile_expert), L.ptr(n_m_tiles), L.c_ll(Mcap), L.c_ll(E * N), bn, L.ptr(st),
                                    L.ptr(push["runs"]), push["peer_ret"], int(push["pairs"]), push["world"], L.stream()),
            "grouped_gemm_mxfp4(push)")
    return None
  if out is None:
    out = torch.empty(Mcap, N, dtype=torch.bfloat16, device=aq.device)
  L.check(L.lib().nmoe_gemm_mxfp4(L.ptr(aq), L.ptr(asf), L.ptr(bq), L.ptr(bsf), L.ptr(out), Mcap, N, K,
                                  L.c_ll(out.stride(0)), 1, E, L.ptr(tile_expert), L.ptr(n_m_tiles), L.c_ll(Mcap),
                                  L.c_ll(E * N), bn, L.ptr(st), None, None, 0, 0, L.stream()), "grouped_gemm_mxfp4")
  return out


def grouped_gemm_mxfp8(aq: torch.Tensor, asf: torch.Tensor, bq: torch.Tensor, bsf: torch.Tensor,
                       tile_expert: torch.Tensor, n_m_tiles: torch.Tensor, *, out: Optional[torch.Tensor] = None,
                       bn: int = 0, push: Optional[dict] = None) -> Optional[torch.Tensor]:
  """Rows of aq [Mcap,K] are 128-aligned expert segments; bq [E,N,K] with stacked scale atoms."""
  Mcap, K = aq.shape
  E, N = bq.size(0), bq.size(1)
  st = status_buffer(aq.device)
  if push is not None:
    L.check(L.lib().nmoe_gemm_mxfp8(L.ptr(aq), L.ptr(asf), L.ptr(bq), L.ptr(bsf), None, Mcap, N, K, L.c_ll(N), 1, E,
                                    L.ptr(tile_expert), L.ptr(n_m_tiles), L.c_ll(Mcap), L.c_ll(E * N), bn, L.ptr(st),
                                    L.ptr(push["runs"]), push["peer_ret"], int(push["pairs"]), push["world"], L.stream()),
            "grouped_gemm_mxfp8(push)")
    return None
  if out is None:
    out = torch.empty(Mcap, N, dtype=torch.bfloat16, device=aq.device)
  L.check(L.lib().nmoe_gemm_mxfp8(L.ptr(aq), L.ptr(asf), L.ptr(bq), L.ptr(bsf), L.ptr(out), Mcap, N, K,
                                  L.c_ll(out.stride(0)), 1, E, L.ptr(tile_expert), L.ptr(n_m_tiles), L.c_ll(Mcap),
                                  L.c_ll(E * N), bn, L.ptr(st), None, None, 0, 0, L.stream()), "grouped_gemm_mxfp8")
  return out


def quant_nvfp4(x: torch.Tensor):
  """x [M,K] bf16 -> (packed E2M1 [M,K/2], UE4M3 scale atoms (one scale per 16 elements), fp32 tensor scale [1]).
  x ~= e2m1 * block_scale * tensor_scale; K % 32 == 0."""
  M, K = x.shape
  # a multiplication (not a division) so that CPU and GPU produce the same bits: x / (scale * ts) lands on
  # exact rounding ties surprisingly often for bf16 inputs, and a 1-ulp difference in ts flips them
  ts = (x.detach().abs().amax().float() * (1.0 / (6.0 * 448.0))).clamp(min=1e-30).reshape(1)
  if not x.is_cuda:
    q, bs, _ = RQ.quant_nvfp4(x.float(), ts)
    Mp = (M + 127) // 128 * 128
    cols = ((K // 16) + 3) // 4 * 4
    sfp = torch.zeros((Mp, cols), dtype=torch.uint8)
    sfp[:M, :K // 16] = bs.view(torch.uint8)
    return q, RQ.sf_to_mma_layout(sfp), ts
  q = torch.empty(M, K // 2, dtype=torch.uint8, device=x.device)
  sf = torch.zeros(sf_bytes(M, 2 * K), dtype=torch.uint8, device=x.device)
  L.check(L.lib().nmoe_quant_nvfp4(L.ptr(x.contiguous()), L.ptr(q), L.ptr(sf), L.c_ll(M), K, L.ptr(ts), L.stream()),
          "quant_nvfp4")
  return q, sf, ts


def gemm_nvfp4(aq: torch.Tensor, asf: torch.Tensor, ats: torch.Tensor, bq: torch.Tensor, bsf: torch.Tensor,
               bts: torch.Tensor, *, out: Optional[torch.Tensor] = None, bn: int = 0) -> torch.Tensor:
  """C[M,N] bf16 = dequant(A) @ dequant(B)^T for NVFP4 operands (E2M1, UE4M3 per 16, fp32 tensor scales) on
  ``kind::mxf4nvf4.block_scale.scale_vec::4X``; the two tensor scales are applied in the epilogue.  K % 64 == 0."""
  M, K = aq.size(0), aq.size(1) * 2
  N = bq.size(0)
  if out is None:
    out = torch.empty(M, N, dtype=torch.bfloat16, device=aq.device)
  alpha = float(ats.item() * bts.item())
  st = status_buffer(aq.device)
  L.check(L.lib().nmoe_gemm_nvfp4(L.ptr(aq), L.ptr(asf), L.ptr(bq), L.ptr(bsf), L.ptr(out), M, N, K,
                                  L.c_ll(out.stride(0)), 0, 1, None, None, L.c_ll(M), L.c_ll(N), bn, L.c_float(alpha),
                                  L.ptr(st), L.stream()), "gemm_nvfp4")
  return out


def swiglu_quant_mxfp4(h13: torch.Tensor, n_tiles: Optional[torch.Tensor] = None):
  """h13 [M,2F] (gate even / up odd) -> silu(gate)*up as MXFP4: (q [M,F/2] nibbles, sf atoms)."""
  M, F2 = h13.shape
  F = F2 // 2
  q = torch.empty(M, F // 2, dtype=torch.uint8, device=h13.device)
  sf = torch.empty(sf_bytes(M, F), dtype=torch.uint8, device=h13.device)
  L.check(L.lib().nmoe_swiglu_quant_mxfp4(L.ptr(h13), L.ptr(q), L.ptr(sf), L.c_ll(M), F, L.ptr(n_tiles), L.stream()),
          "swiglu_quant_mxfp4")
  return q, sf


def grouped_gemm_swiglu_quant(aq: torch.Tensor, asf: torch.Tensor, bq: torch.Tensor, bsf: torch.Tensor,
                              tile_expert: torch.Tensor, n_m_tiles: torch.Tensor, *, fp4: bool = False, bn: int = 0,
                              want_h13: bool = False):
  """Grouped up/gate projection whose epilogue applies SwiGLU and re-quantises: returns the quantised
  activation (E4M3 [Mcap,F] or E2M1 [Mcap,F/2]) and its scale atoms.  The bf16 H13 is not written unless
  ``want_h13`` (then it is returned as a third value, stored by the same epilogue pass).
  ``bq`` = W13 [E, 2F, K(/2)] with gate / up rows interleaved."""
  Mcap = aq.size(0)
  K = aq.size(1) * (2 if fp4 else 1)
  E, N = bq.size(0), bq.size(1)
  F = N // 2
  q = torch.empty(Mcap, F // 2 if fp4 else F, dtype=torch.uint8, device=aq.device)
  sf = torch.empty(sf_bytes(Mcap, F), dtype=torch.uint8, device=aq.device)
  if (F // 32) % 4:
    sf.fill_(127)            # partial last atom: padding scale bytes must be valid
  st = status_buffer(aq.device)
  h13 = torch.empty(Mcap, N, dtype=torch.bfloat16, device=aq.device) if want_h13 else None
  L.check(L.lib().nmoe_gemm_mx_swiglu_quant_h13(L.ptr(aq), L.ptr(asf), L.ptr(bq), L.ptr(bsf), L.ptr(q), L.ptr(sf),
                                                L.ptr(h13), Mcap, N, K, E, L.ptr(tile_expert), L.ptr(n_m_tiles),
                                                L.c_ll(Mcap), L.c_ll(E * N), int(fp4), bn, L.ptr(st), L.stream()),
          "grouped_gemm_swiglu_quant")
  return (q, sf, h13) if want_h13 else (q, sf)


def is_fp4(profile: str) -> bool:
  """The reference's "nvfp4" profile is E2M1 values with one E8M0 scale per 32 elements
  (nmoe/quant.py:45-72), i.e. the OCP MXFP4 format; both names select it here."""
  return profile in ("nvfp4", "mxfp4", "fp4")


class ExpertWeightCache:
  """Block-scaled (MXFP8 or MXFP4) copies of one layer's expert weights.

  The copies are rebuilt whenever the bf16 masters change (version counters), and the expert AdamW
  refreshes them for free: the cache registers itself on the two parameters, and
  ``expert_adamw_quant_`` writes the quantised NEW weights in the same pass that updates them
  (the reference's fused kernel does the same, nmoe/csrc/adamw.cu:73-489 and nmoe/opt.py:118-125)."""

  def __init__(self, profile: str = "fp8"):
    self.fp4 = is_fp4(profile)
    self.ver = [-1, -1]
    self.q = [None, None]        # 2-D views [E*rows, K(/2)]
    self.sf = [None, None]
    self.shape = [None, None]

  def _quantise(self, idx: int, W: torch.Tensor) -> None:
    E, n, k = W.shape
    q, sf = (quant_mxfp4 if self.fp4 else quant_mxfp8)(W.detach().view(E * n, k))
    if self.q[idx] is None or self.q[idx].shape != q.shape:
      self.q[idx], self.sf[idx] = q, sf
    else:
      self.q[idx].copy_(q); self.sf[idx].copy_(sf)
    self.shape[idx] = (E, n, q.size(1))
    self.ver[idx] = W._version
    W._nmoe_qcache = (self, idx)

  def target(self, idx: int):
    """(values [rows, K(/2)], scale atoms, fp4) that a fused optimizer step should overwrite."""
    return self.q[idx], self.sf[idx], self.fp4

  def mark_fresh(self, idx: int, version: int) -> None:
    self.ver[idx] = version

  @torch.no_grad()
  def get(self, W13: torch.Tensor, W2: torch.Tensor):
    for idx, W in ((0, W13), (1, W2)):
      if self.q[idx] is None or self.ver[idx] != W._version:
        self._quantise(idx, W)
    return self.q[0].view(self.shape[0]), self.sf[0], self.q[1].view(self.shape[1]), self.sf[1]


def expert_adamw_quant_(p: torch.Tensor, g: torch.Tensor, m: torch.Tensor, v: torch.Tensor, q: torch.Tensor, sf: torch.Tensor,
                        fp4: bool, *, lr: float, beta1: float, beta2: float, eps: float, weight_decay: float, step: int,
                        grad_scale: float = 1.0) -> None:
  """AdamW on a stack of expert matrices p [E, n, K] (bf16 p / g / m / v) that also writes the block-scaled
  copy of the updated weights into (q, sf)."""
  K = p.size(-1)
  rows = p.numel() // K
  assert p.is_contiguous() and g.is_contiguous() and m.is_contiguous() and v.is_contiguous() and g.dtype == p.dtype
  L.check(L.lib().nmoe_expert_adamw_quant(L.ptr(p), L.ptr(g), L.ptr(m), L.ptr(v), L.c_ll(rows), K, L.c_float(lr),
                                          L.c_float(beta1), L.c_float(beta2), L.c_float(eps), L.c_float(weight_decay),
                                          int(step), L.c_float(grad_scale), L.ptr(q), L.ptr(sf), int(fp4), L.stream()),
          "expert_adamw_quant")


# ------------------------------------------------------------------ NVFP4 proper (16-element blocks, UE4M3 scales)
# A second 4-bit expert profile next to the reference's "nvfp4" (which is E2M1 with one E8M0 scale per 32 elements):
# NVIDIA's NVFP4, E2M1 values with one UE4M3 scale per 16 elements and an fp32 scale per tensor.  Activations use a
# FIXED tensor scale (rows of one expert segment come from different ranks, and post-norm activations are O(1): with
# 1/64 a block maximum between 1.8e-4 and 42 is representable), weights a scale from their own maximum, kept on the
# device; the product reaches the GEMM epilogue through a device pointer, so the layer has no host read.
NVFP4_PROFILE = "nvfp4x16"
NVFP4_ACT_SCALE = 1.0 / 64.0


def nvfp4_act_scale(device) -> torch.Tensor:
  t = _ACT_SCALE.get(device)
  if t is None:
    t = torch.full((1,), NVFP4_ACT_SCALE, dtype=torch.float32, device=device)
    _ACT_SCALE[device] = t
  return t


_ACT_SCALE: dict = {}


def quant_nvfp4_rows(x: torch.Tensor, ts: torch.Tensor):
  """x [M,K] bf16 -> (E2M1 nibbles [M,K/2], UE4M3 scale atoms) against the given tensor scale ``ts`` (fp32 [1], on the
  device): no reduction over x, so rows that hold stale data cannot disturb the others."""
  M, K = x.shape
  if not x.is_cuda:
    q, bs, _ = RQ.quant_nvfp4(x.float(), ts)
    Mp = (M + 127) // 128 * 128
    cols = ((K // 16) + 3) // 4 * 4
    sfp = torch.zeros((Mp, cols), dtype=torch.uint8)
    sfp[:M, :K // 16] = bs.view(torch.uint8)
    return q, RQ.sf_to_mma_layout(sfp)
  q = torch.empty(M, K // 2, dtype=torch.uint8, device=x.device)
  sf = torch.zeros(sf_bytes(M, 2 * K), dtype=torch.uint8, device=x.device)
  L.check(L.lib().nmoe_quant_nvfp4(L.ptr(x.contiguous()), L.ptr(q), L.ptr(sf), L.c_ll(M), K, L.ptr(ts), L.stream()),
          "quant_nvfp4")
  return q, sf


def grouped_gemm_nvfp4(aq: torch.Tensor, asf: torch.Tensor, bq: torch.Tensor, bsf: torch.Tensor, alpha_dev: torch.Tensor,
                       tile_expert: torch.Tensor, n_m_tiles: torch.Tensor, *, out: Optional[torch.Tensor] = None,
                       bn: int = 0) -> torch.Tensor:
  """Rows of aq [Mcap, K/2] are 128-aligned expert segments; bq [E, N, K/2] with stacked UE4M3 scale atoms;
  ``alpha_dev`` (fp32 [1] on the device) = product of the two tensor scales.  Returns bf16 [Mcap, N]."""
  Mcap, K = aq.size(0), aq.size(1) * 2
  E, N = bq.size(0), bq.size(1)
  if out is None:
    out = torch.empty(Mcap, N, dtype=torch.bfloat16, device=aq.device)
  st = status_buffer(aq.device)
  L.check(L.lib().nmoe_gemm_nvfp4_dev(L.ptr(aq), L.ptr(asf), L.ptr(bq), L.ptr(bsf), L.ptr(out), Mcap, N, K,
                                      L.c_ll(out.stride(0)), 1, E, L.ptr(tile_expert), L.ptr(n_m_tiles), L.c_ll(Mcap),
                                      L.c_ll(E * N), bn, L.c_float(1.0), L.ptr(alpha_dev), L.ptr(st), L.stream()),
          "grouped_gemm_nvfp4")
  return out


class ExpertWeightCacheNV16:
  """NVFP4 copies of one layer's expert weights: (W13q, W13sf, alpha13, W2q, W2sf, alpha2) with alpha = weight tensor
  scale x the fixed activation scale, all on the device.  Rebuilt when the bf16 masters change (version counters)."""

  def __init__(self):
    self.ver = [-1, -1]
    self.q = [None, None]
    self.sf = [None, None]
    self.alpha = [None, None]

  @torch.no_grad()
  def get(self, W13: torch.Tensor, W2: torch.Tensor):
    for idx, W in ((0, W13), (1, W2)):
      if self.q[idx] is None or self.ver[idx] != W._version:
        E, n, k = W.shape
        w2d = W.detach().view(E * n, k)
        ts = (w2d.abs().amax().float() * (1.0 / (6.0 * 448.0))).clamp(min=1e-30).reshape(1)
        q, sf = quant_nvfp4_rows(w2d, ts)
        self.q[idx], self.sf[idx] = q.view(E, n, k // 2), sf
        self.alpha[idx] = ts * NVFP4_ACT_SCALE
        self.ver[idx] = W._version
    return self.q[0], self.sf[0], self.alpha[0], self.q[1], self.sf[1], self.alpha[1]
