"""Lightning-indexer scores of DeepSeek sparse attention (reference nmoe/attention/dsa.py:18-319 and its Triton
kernels in nmoe/triton/dsa.py):

    I[b,t,s] = sum_h w[b,t,h] * relu(q_idx[b,t,h,:] . k_idx[b,s,:])        (-inf for s > t when causal)

On a GPU the forward is one tcgen05 GEMM per batch element whose epilogue applies relu, the head weights and the
sum over heads, so the [T, heads, S] logits never reach memory (keys are the rows of the tile: one thread owns one
key and adds up the heads of a query in registers).  The backward recomputes the logits in query chunks with
plain matmuls; the indexer is small (a few heads of 64 dims) and its gradient is not on the critical path.
"""
from __future__ import annotations

import torch

from . import _lib as L
from .tc_gemm import status_buffer


def indexer_scores_ref(q_idx: torch.Tensor, k_idx: torch.Tensor, w: torch.Tensor, causal: bool = True) -> torch.Tensor:
  """fp32 statement of the op: q_idx [B,T,Hi,D], k_idx [B,S,D], w [B,T,Hi] -> [B,T,S]."""
  s = torch.relu(torch.einsum("bthd,bsd->bths", q_idx.float(), k_idx.float()))
  s = (w.float().unsqueeze(-1) * s).sum(2)
  if causal:
    T, S = s.shape[1:]
    s = s.masked_fill(torch.triu(torch.ones(T, S, dtype=torch.bool, device=s.device), 1), float("-inf"))
  return s


def _fused_ok(q_idx: torch.Tensor, k_idx: torch.Tensor) -> bool:
  Hi, D = q_idx.shape[-2:]
  return (q_idx.is_cuda and q_idx.dtype == torch.bfloat16 and k_idx.dtype == torch.bfloat16
          and Hi <= 128 and (Hi & (Hi - 1)) == 0 and D % 8 == 0)


def _forward_fused(q_idx: torch.Tensor, k_idx: torch.Tensor, w: torch.Tensor, causal: bool) -> torch.Tensor:
  B, T, Hi, D = q_idx.shape
  S = k_idx.size(1)
  q2 = q_idx.contiguous().view(B, T * Hi, D)
  k2 = k_idx.contiguous()
  w2 = w.float().contiguous().view(B, T * Hi)
  out = torch.empty(B, T, S, dtype=torch.float32, device=q_idx.device)
  st = status_buffer(q_idx.device)
  for b in range(B):
    L.check(L.lib().nmoe_dsa_indexer_scores(
      L.ptr(k2[b]), L.ptr(q2[b]), L.ptr(w2[b]), L.ptr(out[b]), S, T, Hi, D, L.c_ll(D), L.c_ll(D), L.c_ll(S),
      int(causal), L.ptr(st), L.stream()), "dsa_indexer_scores")
  return out


class _IndexerScores(torch.autograd.Function):
  @staticmethod
  def forward(ctx, q_idx, k_idx, w, causal):
    ctx.save_for_backward(q_idx, k_idx, w)
    return _forward_fused(q_idx, k_idx, w, causal)

  @staticmethod
  def backward(ctx, d_scores):
    q_idx, k_idx, w = ctx.saved_tensors
    return (*indexer_scores_backward(q_idx, k_idx, w, d_scores), None)


def indexer_scores_backward(q_idx: torch.Tensor, k_idx: torch.Tensor, w: torch.Tensor, d_scores: torch.Tensor):
  """Gradients of ``indexer_scores`` w.r.t. (q_idx, k_idx, w) for d_scores [B,T,S]; logits recomputed in query chunks.
  Masked positions must carry zero (non-finite entries are treated as zero)."""
  B, T, Hi, D = q_idx.shape
  d_scores = torch.nan_to_num(d_scores.float(), nan=0.0, posinf=0.0, neginf=0.0)
  kf = k_idx.float()
  dq = torch.empty_like(q_idx, dtype=torch.float32)
  dw = torch.empty(B, T, Hi, dtype=torch.float32, device=q_idx.device)
  dk = torch.zeros_like(kf)
  chunk = max(1, min(T, (1 << 26) // max(1, Hi * k_idx.size(1))))     # bounds the [chunk, Hi, S] logits to 256 MB
  for t0 in range(0, T, chunk):
    t1 = min(T, t0 + chunk)
    qf = q_idx[:, t0:t1].float()
    pre = torch.einsum("bthd,bsd->bths", qf, kf)
    g = d_scores[:, t0:t1].unsqueeze(2)                                # [B,c,1,S]
    dw[:, t0:t1] = (torch.relu(pre) * g).sum(-1)
    dpre = (pre > 0).float() * g * w[:, t0:t1].float().unsqueeze(-1)
    dq[:, t0:t1] = torch.einsum("bths,bsd->bthd", dpre, kf)
    dk += torch.einsum("bths,bthd->bsd", dpre, qf)
  return dq.to(q_idx.dtype), dk.to(k_idx.dtype), dw.to(w.dtype)


def indexer_scores(q_idx: torch.Tensor, k_idx: torch.Tensor, w: torch.Tensor, causal: bool = True) -> torch.Tensor:
  """[B,T,S] fp32 indexer scores; the fused kernel on a GPU with bf16 inputs, the fp32 statement otherwise."""
  if _fused_ok(q_idx, k_idx):
    return _IndexerScores.apply(q_idx, k_idx, w, causal)
  return indexer_scores_ref(q_idx, k_idx, w, causal)
