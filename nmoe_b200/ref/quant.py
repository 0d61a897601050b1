"""Bit-exact emulation of the block-scaled formats in plain PyTorch (CPU oracle).

Contracts (reference: nmoe/csrc/ptx.cu:41-53,118-135; nmoe/csrc/quant.cu:118-250;
nmoe/csrc/swizzle.cuh:33-54):
  * E8M0 scale byte b decodes to 2**(b-127); the encoder picks the smallest power
    of two >= amax/qmax (exponent rounded UP when the mantissa is non-zero),
    clamped to [0, 254]; an all-zero block gets byte 127 (1.0)... any byte works
    for zeros, we use the minimum normal exponent rule below.
  * E4M3 (qmax 448) and E2M1 (qmax 6) values are round-to-nearest-even, saturating.
  * fp8 rows hold 1 value per byte; fp4 rows hold two nibbles per byte, low nibble
    = even element.
  * NVFP4-16 uses 16-element blocks with an unsigned E4M3 scale per block and one
    fp32 tensor scale.
  * MMA scale-factor layout: 128-row x 4-column atoms of 512 bytes, offset inside
    an atom = (m % 32) * 16 + ((m / 32) % 4) * 4 + (k % 4); atoms are laid out
    row-major over (m / 128, k / 4).
"""
from __future__ import annotations

from typing import Tuple

import torch

FP8_MAX = 448.0
FP4_MAX = 6.0
_E2M1_VALUES = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])


def e8m0_encode(amax: torch.Tensor, qmax: float) -> torch.Tensor:
  """uint8 exponent byte: smallest power of two >= amax / qmax."""
  r = (amax.float() / qmax).clamp(min=0.0)
  bits = r.contiguous().view(torch.int32)
  exp = (bits >> 23) & 0xFF
  man = bits & 0x7FFFFF
  e = exp + (man != 0).to(torch.int32)
  e = torch.where(exp == 0, torch.zeros_like(e) + (man != 0).to(torch.int32), e)  # subnormal -> 2^-126
  e = e.clamp(0, 254)
  e = torch.where(r == 0, torch.full_like(e, 127), e)
  return e.to(torch.uint8)


def e8m0_decode(b: torch.Tensor) -> torch.Tensor:
  return torch.pow(2.0, b.to(torch.float32) - 127.0)


def round_e4m3(x: torch.Tensor) -> torch.Tensor:
  """Saturating round-to-nearest-even to E4M3 (fn: no inf, max 448); returns fp32."""
  return x.float().clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn).float()


def round_e2m1(x: torch.Tensor) -> torch.Tensor:
  """Saturating RNE to E2M1 {0,.5,1,1.5,2,3,4,6}; returns fp32."""
  xf = x.float()
  a = xf.abs().clamp(max=FP4_MAX)
  vals = _E2M1_VALUES.to(a.device)
  # midpoints; ties go to the value with an even mantissa bit (codes 0,2,4,6 => 0,1,2,4)
  idx = torch.bucketize(a, (vals[1:] + vals[:-1]) / 2, right=False)
  mid = (vals[1:] + vals[:-1]) / 2
  on_tie = torch.zeros_like(a, dtype=torch.bool)
  for i in range(7):
    on_tie |= (a == mid[i])
  # bucketize(right=False) sends a==mid[i] to index i (lower value). For a tie pick even code.
  lower = idx
  tie_up = on_tie & ((lower % 2) == 1)
  idx = torch.where(tie_up, lower + 1, lower)
  return torch.sign(xf) * vals[idx.clamp(max=7)]


def e2m1_code(x_rounded: torch.Tensor) -> torch.Tensor:
  """4-bit code (sign<<3 | magnitude index) of an already-rounded E2M1 value."""
  vals = _E2M1_VALUES.to(x_rounded.device)
  mag = torch.bucketize(x_rounded.abs(), vals, right=False).clamp(max=7)
  sign = (torch.signbit(x_rounded)).to(torch.int32)
  return (sign << 3 | mag.to(torch.int32)).to(torch.uint8)


def e2m1_decode(code: torch.Tensor) -> torch.Tensor:
  vals = _E2M1_VALUES.to(code.device)
  c = code.to(torch.int64)
  v = vals[c & 7]
  return torch.where((c & 8) != 0, -v, v)


def quant_mxfp8(x: torch.Tensor, block: int = 32) -> Tuple[torch.Tensor, torch.Tensor]:
  """[M,K] -> (float8_e4m3fn [M,K], uint8 E8M0 scales [M,K/block], row-major)."""
  M, K = x.shape
  xb = x.float().view(M, K // block, block)
  sf = e8m0_encode(xb.abs().amax(-1), FP8_MAX)
  q = round_e4m3(xb / e8m0_decode(sf).unsqueeze(-1)).view(M, K)
  return q.to(torch.float8_e4m3fn), sf


def dequant_mxfp8(q: torch.Tensor, sf: torch.Tensor, block: int = 32) -> torch.Tensor:
  M, K = q.shape
  return (q.float().view(M, K // block, block) * e8m0_decode(sf).unsqueeze(-1)).view(M, K)


def quant_mxfp4(x: torch.Tensor, block: int = 32) -> Tuple[torch.Tensor, torch.Tensor]:
  """[M,K] -> (uint8 packed [M,K/2], uint8 E8M0 scales [M,K/block])."""
  M, K = x.shape
  xb = x.float().view(M, K // block, block)
  sf = e8m0_encode(xb.abs().amax(-1), FP4_MAX)
  r = round_e2m1(xb / e8m0_decode(sf).unsqueeze(-1)).view(M, K)
  c = e2m1_code(r)
  return (c[:, 0::2] | (c[:, 1::2] << 4)).contiguous(), sf


def dequant_mxfp4(packed: torch.Tensor, sf: torch.Tensor, block: int = 32) -> torch.Tensor:
  M, Kh = packed.shape
  c = torch.stack((packed & 0xF, packed >> 4), dim=-1).view(M, Kh * 2)
  v = e2m1_decode(c)
  return (v.view(M, -1, block) * e8m0_decode(sf).unsqueeze(-1)).view(M, Kh * 2)


def quant_nvfp4(x: torch.Tensor, ts: torch.Tensor | None = None) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
  """True NVFP4: 16-element blocks, E4M3 block scales, one fp32 tensor scale.

  Returns (uint8 packed [M,K/2], float8_e4m3fn scales [M,K/16], fp32 tensor scale).
  x ~= e2m1 * block_scale * tensor_scale.
  """
  M, K = x.shape
  xf = x.float()
  if ts is None:
    ts = (xf.abs().amax() / (FP4_MAX * FP8_MAX)).clamp(min=1e-30)
  ts = ts.reshape(()).float()
  xb = xf.view(M, K // 16, 16)
  bs = (xb.abs().amax(-1) / FP4_MAX / ts).clamp(max=FP8_MAX).to(torch.float8_e4m3fn)
  denom = (bs.float() * ts).unsqueeze(-1)
  r = round_e2m1(torch.where(denom > 0, xb / denom, torch.zeros_like(xb))).view(M, K)
  c = e2m1_code(r)
  return (c[:, 0::2] | (c[:, 1::2] << 4)).contiguous(), bs, ts


def dequant_nvfp4(packed: torch.Tensor, bs: torch.Tensor, ts: torch.Tensor) -> torch.Tensor:
  M, Kh = packed.shape
  c = torch.stack((packed & 0xF, packed >> 4), dim=-1).view(M, Kh * 2)
  return (e2m1_decode(c).view(M, -1, 16) * (bs.float() * ts).unsqueeze(-1)).view(M, Kh * 2)


def sf_mma_offset(m: torch.Tensor, k: torch.Tensor, sf_k: int) -> torch.Tensor:
  """Byte offset of scale (row m, scale column k) in the MMA atom layout; sf_k = padded #columns (multiple of 4)."""
  atom = (m // 128) * (sf_k // 4) + (k // 4)
  return atom * 512 + (m % 32) * 16 + ((m // 32) % 4) * 4 + (k % 4)


def sf_to_mma_layout(sf: torch.Tensor) -> torch.Tensor:
  """Row-major [M, sf_k] (M multiple of 128, sf_k multiple of 4) -> flat uint8 buffer in MMA atom layout."""
  M, sk = sf.shape
  assert M % 128 == 0 and sk % 4 == 0
  m = torch.arange(M).unsqueeze(1).expand(M, sk)
  k = torch.arange(sk).unsqueeze(0).expand(M, sk)
  out = torch.empty(M * sk, dtype=sf.dtype)
  out[sf_mma_offset(m, k, sk).reshape(-1)] = sf.reshape(-1).cpu()
  return out


def sf_from_mma_layout(buf: torch.Tensor, M: int, sk: int) -> torch.Tensor:
  m = torch.arange(M).unsqueeze(1).expand(M, sk)
  k = torch.arange(sk).unsqueeze(0).expand(M, sk)
  return buf.cpu()[sf_mma_offset(m, k, sk).reshape(-1)].view(M, sk)
