"""Kimi Delta Attention: gated delta-rule linear attention on MLA-style projections
(reference nmoe/attention/kda.py:20-76 and the chunked kernels in nmoe/triton/kda.py).

Per head, with L2-normalised q and k, per-key-channel log-decay g_t <= 0 and write strength
beta_t in (0,1), the state S [Dk, Dv] evolves as
    S <- diag(exp(g_t)) S ;  S <- S + beta_t k_t (v_t - S^T k_t)^T ;  o_t = S^T (q_t / sqrt(Dk))
``kda_recurrent`` is that recurrence token by token; ``kda_chunked`` processes ``chunk`` tokens at a
time with the WY / UT-transform form (matrix products inside a chunk, one state update per chunk) as a
plain PyTorch loop: the oracle, and the path for CPU tensors.  On a GPU the layer uses
``ops.kda.kda_chunk_scan``: the same transform batched over all chunks, with the recurrence over
chunks (forward and backward) on the scan kernel in ``csrc/kda.cu``."""
from __future__ import annotations

import torch
from ..init import trunc_normal_
import torch.nn.functional as F
from torch import nn

from ... import ops
from ..norm import RMSNorm


def _l2norm(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
  return x * torch.rsqrt(x.pow(2).sum(-1, keepdim=True) + eps)


def kda_recurrent(q, k, v, g, beta, scale=None):
  """q,k,g [B,T,H,Dk]; v [B,T,H,Dv]; beta [B,T,H] -> o [B,T,H,Dv] (fp32 math)."""
  B, T, H, Dk = q.shape
  scale = Dk ** -0.5 if scale is None else scale
  q, k = _l2norm(q.float()) * scale, _l2norm(k.float())
  v, g, beta = v.float(), g.float(), beta.float()
  S = q.new_zeros(B, H, Dk, v.size(-1))
  out = []
  for t in range(T):
    S = S * torch.exp(g[:, t]).unsqueeze(-1)
    err = v[:, t] - torch.einsum("bhk,bhkv->bhv", k[:, t], S)
    S = S + torch.einsum("bhk,bhv->bhkv", k[:, t] * beta[:, t].unsqueeze(-1), err)
    out.append(torch.einsum("bhk,bhkv->bhv", q[:, t], S))
  return torch.stack(out, 1)


def kda_chunked(q, k, v, g, beta, scale=None, chunk: int = 64):
  """Same function as ``kda_recurrent`` evaluated chunk by chunk."""
  B, T, H, Dk = q.shape
  Dv = v.size(-1)
  scale = Dk ** -0.5 if scale is None else scale
  pad = (-T) % chunk
  if pad:
    z = lambda x: F.pad(x, (0, 0) * (x.dim() - 2) + (0, pad))
    q, k, v, g = (F.pad(x, (0, 0, 0, 0, 0, pad)) for x in (q, k, v, g))
    beta = F.pad(beta, (0, 0, 0, pad))
  Tp = T + pad
  n = Tp // chunk
  f = lambda x: x.float().view(B, n, chunk, H, -1).permute(0, 3, 1, 2, 4)       # [B,H,n,C,D]
  q, k, v, g = f(_l2norm(q.float()) * scale), f(_l2norm(k.float())), f(v), f(g)
  beta = beta.float().view(B, n, chunk, H).permute(0, 3, 1, 2)
  gc = g.cumsum(3)                                                             # decay from chunk start, per channel
  S = q.new_zeros(B, H, Dk, Dv)
  outs = []
  eye = torch.eye(chunk, device=q.device)
  strict = torch.tril(torch.ones(chunk, chunk, device=q.device), -1)
  incl = torch.tril(torch.ones(chunk, chunk, device=q.device))
  for c in range(n):
    qc, kc, vc, gcc, bc = q[:, :, c], k[:, :, c], v[:, :, c], gc[:, :, c], beta[:, :, c]
    kd = kc * torch.exp(gcc)            # k_i scaled to "chunk start" coordinates for reading the incoming state
    ki = kc * torch.exp(-gcc)           # k_j expressed so that (kd_i . ki_j) carries decay from j to i
    A = torch.einsum("bhik,bhjk->bhij", kd, ki) * strict                      # k_i^T Decay(j->i) k_j, j < i
    # (I + diag(beta) A) W = diag(beta) (V - Kd S)   solves the in-chunk delta-rule dependencies
    M = eye + bc.unsqueeze(-1) * A
    rhs = bc.unsqueeze(-1) * (vc - torch.einsum("bhik,bhkv->bhiv", kd, S))
    W = torch.linalg.solve_triangular(M, rhs, upper=False)                    # effective written values
    qd = qc * torch.exp(gcc)
    o = torch.einsum("bhik,bhkv->bhiv", qd, S) + torch.einsum("bhij,bhjv->bhiv", torch.einsum("bhik,bhjk->bhij", qd, ki) * incl, W)
    outs.append(o)
    g_end = gcc[:, :, -1]                                                     # [B,H,Dk]
    S = S * torch.exp(g_end).unsqueeze(-1) + torch.einsum("bhjk,bhjv->bhkv", ki * torch.exp(g_end).unsqueeze(2), W)
  o = torch.stack(outs, 2).reshape(B, H, Tp, Dv).permute(0, 2, 1, 3)
  return o[:, :T]


class KDA(nn.Module):
  def __init__(self, cfg, dtype: torch.dtype = torch.bfloat16):
    super().__init__()
    self.dim, self.n_heads = cfg.dim, cfg.n_heads
    self.nope, self.rope_dim, self.v_dim = cfg.qk_nope_head_dim, cfg.qk_rope_head_dim, cfg.v_head_dim
    self.qk_dim = self.nope + self.rope_dim
    self.q_lora_rank, self.kv_lora_rank = cfg.q_lora_rank, cfg.kv_lora_rank
    self.chunk = int((cfg.attn_kda or {}).get("chunk", 64))
    mk = lambda o, i: nn.Parameter(torch.empty(o, i, dtype=dtype))
    self.wq_a, self.wq_b = mk(self.q_lora_rank, self.dim), mk(self.n_heads * self.qk_dim, self.q_lora_rank)
    self.q_norm = RMSNorm(self.q_lora_rank, cfg.rms_norm_eps, dtype)
    self.wkv_a = mk(self.kv_lora_rank + self.rope_dim, self.dim)
    self.kv_norm = RMSNorm(self.kv_lora_rank, cfg.rms_norm_eps, dtype)
    self.wkv_b = mk(self.n_heads * (self.nope + self.v_dim), self.kv_lora_rank)
    self.wo = mk(self.dim, self.n_heads * self.v_dim)
    self.wg, self.wg_b = mk(self.n_heads * self.qk_dim, self.dim), nn.Parameter(torch.zeros(self.n_heads * self.qk_dim, dtype=dtype))
    self.wb = mk(self.n_heads, self.dim)
    self.window = 0

  def init_weights(self, init_std: float = 0.02) -> None:
    for w in (self.wq_a, self.wq_b, self.wkv_a, self.wkv_b, self.wg, self.wb):
      trunc_normal_(w, mean=0.0, std=0.02)
    nn.init.zeros_(self.wg_b)
    trunc_normal_(self.wo, mean=0.0, std=init_std)
    self.q_norm.weight.data.fill_(1.0)
    self.kv_norm.weight.data.fill_(1.0)

  def forward(self, x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    B, T, _ = x.shape
    h = self.n_heads
    q = ops.linear(self.q_norm(ops.linear(x, self.wq_a)), self.wq_b).view(B, T, h, self.qk_dim)
    kv_a = ops.linear(x, self.wkv_a)
    lat, k_pe = torch.split(kv_a, [self.kv_lora_rank, self.rope_dim], dim=-1)
    kv = ops.linear(self.kv_norm(lat.contiguous()), self.wkv_b).view(B, T, h, self.nope + self.v_dim)
    k = torch.cat((kv[..., :self.nope], k_pe.unsqueeze(2).expand(B, T, h, self.rope_dim)), -1)
    g = F.logsigmoid(ops.linear(x, self.wg, self.wg_b).float()).view(B, T, h, self.qk_dim)
    beta = torch.sigmoid(ops.linear(x, self.wb).float()).view(B, T, h)
    if x.is_cuda and self.chunk == 64 and self.v_dim % 64 == 0 and self.qk_dim % 4 == 0 and self.qk_dim <= 256:
      # batched WY transform + the chunk recurrence on the CUDA scan kernel (csrc/kda.cu), forward and backward
      from ...ops.kda import kda_chunk_scan
      o = kda_chunk_scan(q, k, kv[..., self.nope:], g, beta)
    else:
      o = kda_chunked(q, k, kv[..., self.nope:], g, beta, chunk=self.chunk)
    o = torch.nan_to_num(o, nan=0.0, posinf=1e4, neginf=-1e4).to(x.dtype)
    return ops.linear(o.reshape(B, T, h * self.v_dim), self.wo)
