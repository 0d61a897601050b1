"""Plain-PyTorch statements of every hot op.  This file is the numerical oracle:
each CUDA kernel in ``nmoe_b200.ops`` is tested against the function of the same
name here, evaluated in fp32.  Everything runs on CPU.

Math follows the reference's eager code: router nmoe/model.py:61-77, MoE loop
tests/test_rdep_accuracy.py:25-55, rotary nmoe/attention/rope.py:7-22, SWA
reference nmoe/triton/swa.py:576-614, masked CE nmoe/train.py:103-105.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
  xf = x.float()
  y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
  return (y * weight.float()).to(x.dtype)


def rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
  """Half-split rotary on the last dim. x: [B, S, h, D]; cos/sin: [S, D/2]."""
  S = x.size(1)
  c = cos[:S].unsqueeze(-2).float()
  s = sin[:S].unsqueeze(-2).float()
  half = x.size(-1) // 2
  x1, x2 = x[..., :half].float(), x[..., half:].float()
  return torch.cat((x1 * c - x2 * s, x2 * c + x1 * s), dim=-1).to(x.dtype)


def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
  return (F.silu(gate.float()) * up.float()).to(gate.dtype)


def router(logits: torch.Tensor, bias: Optional[torch.Tensor], topk: int, *, route_scale: float = 1.0,
           kind: str = "sigmoid", n_groups: int = 0, max_groups: int = 0) -> Tuple[torch.Tensor, torch.Tensor]:
  """Top-k routing.  Returns (weights fp32 [T,K], expert ids int64 [T,K]).

  sigmoid: scale the logits, sigmoid, select on score+bias, weight = unbiased
  score renormalised over the selected k.  softmax: softmax over experts, select
  on prob(+bias), weights are the selected probabilities (renormalised).
  ``max_groups`` > 0 restricts each token to the ``max_groups`` expert groups
  (of ``n_groups`` equal groups, i.e. devices) with the highest group maximum.
  """
  lf = logits.float() * route_scale
  scores = torch.sigmoid(lf) if kind == "sigmoid" else torch.softmax(lf, dim=-1)
  sel = scores if bias is None else scores + bias.float()
  if max_groups > 0 and n_groups > 1:
    T, E = sel.shape
    g = sel.view(T, n_groups, E // n_groups).amax(-1)
    keep = torch.topk(g, k=max_groups, dim=-1).indices
    mask = torch.zeros(T, n_groups, dtype=torch.bool, device=sel.device).scatter_(1, keep, True)
    mask = mask.unsqueeze(-1).expand(T, n_groups, E // n_groups).reshape(T, E)
    sel = sel.masked_fill(~mask, float("-inf"))
  idx = torch.topk(sel, k=topk, dim=-1).indices
  w = torch.gather(scores, 1, idx)
  w = w / w.sum(-1, keepdim=True).clamp(min=1e-12)
  return w, idx


def expert_mlp(x: torch.Tensor, w1: torch.Tensor, w3: torch.Tensor, w2: torch.Tensor) -> torch.Tensor:
  """One expert: (silu(x@w1) * (x@w3)) @ w2 with w1,w3 [H,Dff], w2 [Dff,H]."""
  return (F.silu(x @ w1) * (x @ w3)) @ w2


def moe(x: torch.Tensor, eid: torch.Tensor, gates: torch.Tensor,
        W1: torch.Tensor, W3: torch.Tensor, W2: torch.Tensor) -> torch.Tensor:
  """out[t] = sum_k gates[t,k] * Expert_{eid[t,k]}(x[t]), accumulated in fp32.

  Per-expert loop; differentiable w.r.t. x, gates and the weights.
  """
  T, H = x.shape
  out = torch.zeros(T, H, dtype=torch.float32, device=x.device)
  for e in range(W1.size(0)):
    tok, slot = torch.nonzero(eid == e, as_tuple=True)
    if tok.numel() == 0:
      continue
    y = expert_mlp(x[tok], W1[e], W3[e], W2[e]).float()
    out = out.index_add(0, tok, y * gates[tok, slot].float().unsqueeze(-1))
  return out.to(x.dtype)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, *, causal: bool = True,
              window: int = 0, sinks: Optional[torch.Tensor] = None) -> torch.Tensor:
  """Eager softmax attention.  q,k: [B,S,Hq|Hkv,Dqk], v: [B,S,Hkv,Dv] -> [B,S,Hq,Dv].

  ``window`` > 0 keeps keys j with i - window < j <= i.  ``sinks`` ([Hq]) adds a
  learned logit per head to the softmax denominator only.  GQA when Hkv < Hq.
  """
  B, S, Hq, _ = q.shape
  Hkv = k.size(2)
  if Hkv != Hq:
    k = k.repeat_interleave(Hq // Hkv, dim=2)
    v = v.repeat_interleave(Hq // Hkv, dim=2)
  s = torch.einsum("bihd,bjhd->bhij", q.float(), k.float()) * scale
  i = torch.arange(S, device=q.device).unsqueeze(-1)
  j = torch.arange(S, device=q.device).unsqueeze(0)
  mask = torch.ones(S, S, dtype=torch.bool, device=q.device)
  if causal:
    mask &= j <= i
  if window > 0:
    mask &= j > i - window
  s = s.masked_fill(~mask, float("-inf"))
  if sinks is not None:
    sk = sinks.float().view(1, Hq, 1, 1).expand(B, Hq, S, 1)
    p = torch.softmax(torch.cat((s, sk), dim=-1), dim=-1)[..., :-1]
  else:
    p = torch.softmax(s, dim=-1)
  return torch.einsum("bhij,bjhd->bihd", p, v.float()).to(q.dtype)


def masked_cross_entropy(logits: torch.Tensor, targets: torch.Tensor, ignore_id: int) -> torch.Tensor:
  """Mean CE over positions whose target differs from ``ignore_id`` (the EOS/pad id)."""
  loss = F.cross_entropy(logits.float().reshape(-1, logits.size(-1)), targets.reshape(-1), reduction="none")
  mask = (targets.reshape(-1) != ignore_id).float()
  return (loss * mask).sum() / mask.sum().clamp(min=1.0)


def lm_head_loss(h: torch.Tensor, w: torch.Tensor, targets: torch.Tensor, ignore_id: int,
                 logit_scale: float) -> torch.Tensor:
  """Masked CE of ``(h @ w.T) * logit_scale`` without exposing the logits."""
  return masked_cross_entropy((h @ w.t()) * logit_scale, targets, ignore_id)


def adamw_step(p: torch.Tensor, g: torch.Tensor, m: torch.Tensor, v: torch.Tensor, *, lr: float, beta1: float,
               beta2: float, eps: float, weight_decay: float, step: int) -> None:
  """Decoupled-decay AdamW in fp32 math, decay applied first, in place."""
  pf, gf, mf, vf = p.float(), g.float(), m.float(), v.float()
  pf = pf * (1.0 - lr * weight_decay)
  mf = beta1 * mf + (1.0 - beta1) * gf
  vf = beta2 * vf + (1.0 - beta2) * gf * gf
  bc1 = 1.0 - beta1 ** step
  bc2 = 1.0 - beta2 ** step
  pf = pf - (lr / bc1) * mf / (vf.sqrt() / math.sqrt(bc2) + eps)
  p.copy_(pf)
  m.copy_(mf)
  v.copy_(vf)


def newton_schulz(x: torch.Tensor, steps: int = 5, coeffs: Tuple[float, float, float] = (3.4445, -4.7750, 2.0315),
                  eps: float = 1e-7) -> torch.Tensor:
  """Muon orthogonaliser: Frobenius-normalise then X <- aX + (bA + cA^2)X, A = X X^T."""
  a, b, c = coeffs
  X = x.float()
  transposed = X.size(-2) > X.size(-1)
  if transposed:
    X = X.transpose(-1, -2)
  X = X / (X.norm(dim=(-2, -1), keepdim=True) + eps)
  for _ in range(steps):
    A = X @ X.transpose(-1, -2)
    X = a * X + (b * A + c * (A @ A)) @ X
  if transposed:
    X = X.transpose(-1, -2)
  return X.to(x.dtype)
