"""Softmax attention entry point: causal, optional sliding window, optional learned sinks, GQA.

q,k: [B,S,Hq|Hkv,Dqk]; v: [B,S,Hkv,Dv] -> [B,S,Hq,Dv].  MLA calls it with (Dqk,Dv)=(192,128).
CPU tensors run the eager oracle.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F

from ..ref import ops as R


def _banded_eager(q, k, v, scale, window, sinks):
  """Query-block tiled eager attention for windows/sinks on CUDA (library GEMMs).

  Each block of ``bq`` queries only sees keys in [start - window + 1, end], so the cost is
  O(S * (bq + window)) instead of O(S^2).
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


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, *, causal: bool = True,
              window: int = 0, sinks: Optional[torch.Tensor] = None) -> torch.Tensor:
  if not q.is_cuda:
    return R.attention(q, k, v, scale, causal=causal, window=window, sinks=sinks)
  if window > 0 or sinks is not None:
    return _banded_eager(q, k, v, scale, window, sinks)
  Hq, Hkv = q.size(2), k.size(2)
  o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=causal,
                                     scale=scale, enable_gqa=(Hq != Hkv))
  return o.transpose(1, 2)
