"""Helpers shared by the sparse / linear attention variants: masked eager attention with GQA and
optional sinks (fp32 softmax), used where the mask is data dependent."""
from __future__ import annotations

from typing import Optional

import torch


def masked_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, allowed: torch.Tensor, scale: float,
                     sinks: Optional[torch.Tensor] = None, q_block: int = 256) -> torch.Tensor:
  """q [B,T,H,D]; k,v [B,S,Hkv,D*]; allowed: bool, broadcastable to [B,H,T,S] (True = may attend).
  Rows with no allowed key give zeros.  Query blocks bound the size of the score tensor."""
  B, T, H, _ = q.shape
  Hkv = k.size(2)
  if Hkv != H:
    k = k.repeat_interleave(H // Hkv, dim=2)
    v = v.repeat_interleave(H // Hkv, dim=2)
  kt, vt = k.transpose(1, 2).float(), v.transpose(1, 2).float()
  outs = []
  for t0 in range(0, T, q_block):
    t1 = min(T, t0 + q_block)
    s = torch.matmul(q[:, t0:t1].transpose(1, 2).float(), kt.transpose(-1, -2)) * scale      # [B,H,t,S]
    m = allowed[..., t0:t1, :] if allowed.size(-2) == T else allowed
    s = s.masked_fill(~m, float("-inf"))
    if sinks is not None:
      s = torch.cat((s, sinks.float().view(1, H, 1, 1).expand(B, H, t1 - t0, 1)), dim=-1)
    mx = s.amax(-1, keepdim=True).clamp(min=-1e30)
    p = torch.exp(s - mx)
    p = p / p.sum(-1, keepdim=True).clamp(min=1e-30)
    if sinks is not None:
      p = p[..., :-1]
    outs.append(torch.matmul(p, vt).transpose(1, 2))
  return torch.cat(outs, dim=1).to(q.dtype)
