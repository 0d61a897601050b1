"""DeepSeek Sparse Attention: MLA whose keys are restricted, per query, to the top-k tokens ranked by
a cheap "lightning indexer" (reference nmoe/attention/dsa.py:18-319).

  indexer score  I[t,s] = sum_j w[t,j] * relu(q_idx[t,j] . k_idx[s])            (few heads, small dim)
  attention      over {s <= t : s in top-k(I[t,:])}
Training modes: ``dense_warmup`` (dense attention; the indexer is trained to match the attention
distribution with a KL loss) and ``sparse`` (attention over the selected tokens; KL on them).
``indexer_alignment_loss()`` is valid after a forward.  The indexer sees detached inputs."""
from __future__ import annotations

import torch
from ..init import trunc_normal_
import torch.nn.functional as F
from torch import nn

from ... import ops
from ...ops.attention import SparseMask
from ...ops.indexer import indexer_scores
from .common import masked_attention
from .mla import MLA


def lightning_indexer(q_idx: torch.Tensor, k_idx: torch.Tensor, w: torch.Tensor, top_k: int, causal: bool = True):
  """q_idx [B,T,Hi,Di], k_idx [B,S,Di], w [B,T,Hi] -> (top scores [B,T,k], indices int32 [B,T,k])."""
  s = indexer_scores(q_idx, k_idx, w, causal)          # fused GEMM + relu + head sum on a GPU
  vals, idx = s.topk(min(top_k, s.size(-1)), dim=-1)
  return vals, idx.to(torch.int32)


class DSA(MLA):
  def __init__(self, cfg, dtype: torch.dtype = torch.bfloat16):
    super().__init__(cfg, dtype)
    o = cfg.attn_dsa or {}
    self.n_idx_heads, self.idx_dim = int(o.get("n_idx_heads", 4)), int(o.get("idx_dim", 64))
    self.top_k, self.training_mode = int(o.get("top_k", 2048)), o.get("training_mode", "sparse")
    mk = lambda a, b: nn.Parameter(torch.empty(a, b, dtype=dtype))
    self.wq_idx, self.wk_idx, self.w_idx = mk(self.n_idx_heads * self.idx_dim, self.dim), mk(self.idx_dim, self.dim), mk(self.n_idx_heads, self.dim)
    self._cache = {}

  def init_weights(self, init_std: float = 0.02) -> None:
    super().init_weights(init_std)
    for w in (self.wq_idx, self.wk_idx, self.w_idx):
      trunc_normal_(w, mean=0.0, std=0.02)

  def _idx_inputs(self, x):
    B, T, _ = x.shape
    return (F.linear(x, self.wq_idx).view(B, T, self.n_idx_heads, self.idx_dim), F.linear(x, self.wk_idx),
            F.linear(x, self.w_idx))

  def _qkv(self, x, cos, sin):
    B, S, _ = x.shape
    h = self.n_heads
    q = ops.linear(self.q_norm(ops.linear(x, self.wq_a)), self.wq_b).view(B, S, h, self.qk_dim)
    q = ops.rope(q, cos, sin, offset=self.nope)
    kv_a = ops.linear(x, self.wkv_a)
    lat, k_pe = torch.split(kv_a, [self.kv_lora_rank, self.rope_dim], dim=-1)
    k_pe = ops.rope(k_pe.reshape(B, S, 1, self.rope_dim), cos, sin)
    kv = ops.linear(self.kv_norm(lat.contiguous()), self.wkv_b).view(B, S, h, self.nope + self.v_dim)
    k = torch.cat((kv[..., :self.nope], k_pe.expand(B, S, h, self.rope_dim)), -1)
    return q, k, kv[..., self.nope:]

  def forward(self, x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    B, T, _ = x.shape
    q, k, v = self._qkv(x, cos, sin)
    eager = self.training_mode == "dense_warmup" or not (x.is_cuda and x.dtype == torch.bfloat16)
    causal = torch.tril(torch.ones(T, T, dtype=torch.bool, device=x.device)).view(1, 1, T, T) if eager else None
    qi, ki, wi = self._idx_inputs(x.detach())
    if self.training_mode == "dense_warmup":
      o = masked_attention(q, k, v, causal, self.softmax_scale)
      dense = indexer_scores(qi, ki, wi, causal=False)
      with torch.no_grad():
        s = torch.einsum("bihd,bjhd->bhij", q.float(), k.float()) * self.softmax_scale
        p = torch.softmax(s.masked_fill(~causal, float("-inf")), -1)
      self._cache = {"mode": "dense", "scores": dense, "attn": p}
    elif x.is_cuda and x.dtype == torch.bfloat16:
      # indexer scores (tcgen05 GEMM with the relu / head-sum epilogue) -> per-query top-k as a packed bit mask
      # (radix select, no sort, no index lists) -> the tcgen05 attention kernels test the bits in their softmax
      # stage, forward and backward: nothing of size [B, H, T, T] exists on this path
      full = indexer_scores(qi, ki, wi, causal=True)
      mask = SparseMask.from_topk_scores(full.detach(), self.top_k)
      o = ops.attention(q, k, v, self.softmax_scale, mask=mask)
      self._cache = {"mode": "sparse", "scores_full": full, "q": q.detach(), "k": k.detach()}
    else:
      scores, sel = lightning_indexer(qi, ki, wi, self.top_k)
      allowed = torch.zeros(B, T, T, dtype=torch.bool, device=x.device)
      allowed.scatter_(2, sel.long(), True)
      o = masked_attention(q, k, v, allowed.unsqueeze(1) & causal, self.softmax_scale)
      self._cache = {"mode": "sparse", "scores": scores, "sel": sel, "q": q.detach(), "k": k.detach()}
    return ops.linear(o.reshape(B, T, self.n_heads * self.v_dim), self.wo)

  def indexer_alignment_loss(self) -> torch.Tensor:
    c = self._cache
    if not c:
      raise RuntimeError("indexer_alignment_loss() must be called after forward()")
    if c["mode"] == "dense":
      scores, p = c["scores"], c["attn"].sum(1)
      B, T, _ = scores.shape
      p = p / (p.sum(-1, keepdim=True) + 1e-8)
      m = torch.triu(torch.ones(T, T, dtype=torch.bool, device=scores.device), 1)
      logq = F.log_softmax(scores.masked_fill(m, float("-inf")), -1)
      kl = F.kl_div(logq.masked_fill(m, 0.0), p.masked_fill(m, 0.0), reduction="none").masked_fill(m, 0.0)
      return kl.sum() / (B * T)
    if "scores_full" in c:      # GPU path: the index lists are only needed here, for the auxiliary loss
      full = c["scores_full"]
      scores, sel = full.topk(min(self.top_k, full.size(-1)), dim=-1)
      c = dict(c, scores=scores, sel=sel)
    scores, sel, q, k = c["scores"], c["sel"].long(), c["q"], c["k"]
    B, T, K = scores.shape
    ks = torch.gather(k.unsqueeze(1).expand(B, T, T, *k.shape[2:]), 2,
                      sel.view(B, T, K, 1, 1).expand(B, T, K, *k.shape[2:]))           # [B,T,K,H,D]
    valid = ~torch.isinf(scores)
    a = torch.einsum("bthd,btkhd->bhtk", q.float(), ks.float()) * self.softmax_scale
    p = torch.softmax(a.masked_fill(~valid.unsqueeze(1), float("-inf")), -1).sum(1)
    p = p / (p.sum(-1, keepdim=True) + 1e-8)
    logq = F.log_softmax(scores.masked_fill(~valid, -1e30), -1)
    kl = F.kl_div(logq, p, reduction="none").masked_fill(~valid, 0.0)
    return kl.sum() / valid.sum().clamp(min=1)
