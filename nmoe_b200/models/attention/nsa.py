"""Native Sparse Attention (arXiv:2502.11089; reference nmoe/attention/nsa.py:20-403).

Three causal paths mixed by per-token sigmoid gates (Eq. 5):
  cmp  attention over keys/values compressed by a learnable MLP over overlapping blocks of
       ``cmp_len`` tokens with stride ``cmp_stride`` (Eq. 7); its probabilities are also aggregated
       into scores of selection blocks of ``slc_block`` tokens (Eq. 8-9)
  slc  attention over the query's own block plus the top ``topk_blocks`` selection blocks (three of
       them fixed: the first block and the two preceding ones), chosen on the scores summed over
       the heads of a KV group (Eq. 10-12)
  swa  sliding-window attention with learned sinks (window set per layer)
"""
from __future__ import annotations

import torch
from ..init import trunc_normal_
from torch import nn

from ... import ops
from ...ops.attention import SparseMask, attention
from .common import masked_attention


class NSA(nn.Module):
  def __init__(self, cfg, dtype: torch.dtype = torch.bfloat16):
    super().__init__()
    self.n_heads, self.head_dim = cfg.n_heads, int(cfg.v_head_dim)
    if cfg.qk_nope_head_dim + cfg.qk_rope_head_dim != self.head_dim:
      raise ValueError("NSA requires qk_nope_head_dim + qk_rope_head_dim == v_head_dim")
    o = cfg.attn_nsa or {}
    self.n_kv_heads = int(o.get("kv_heads", (cfg.attn_swa or {}).get("kv_heads", self.n_heads)))
    if self.n_heads % self.n_kv_heads:
      raise ValueError("NSA requires n_heads % kv_heads == 0")
    self.G = self.n_heads // self.n_kv_heads
    self.cmp_len, self.cmp_stride = int(o.get("cmp_len", 32)), int(o.get("cmp_stride", 16))
    self.slc_block, self.topk = int(o.get("slc_block", 64)), int(o.get("topk_blocks", 16))
    self.window = 0
    self.softmax_scale = self.head_dim ** -0.5
    D, H, KV = self.head_dim, self.n_heads, self.n_kv_heads
    mk = lambda *s: nn.Parameter(torch.empty(*s, dtype=dtype))
    self.qkv_w, self.qkv_b = mk((H + 2 * KV) * D, cfg.dim), nn.Parameter(torch.zeros((H + 2 * KV) * D, dtype=dtype))
    self.out_w, self.out_b = mk(cfg.dim, H * D), nn.Parameter(torch.zeros(cfg.dim, dtype=dtype))
    self.sinks = nn.Parameter(torch.zeros(H, dtype=dtype))
    ch = int(o.get("cmp_hidden", 2 * D))
    self.cmp_pos = nn.Parameter(torch.zeros(self.cmp_len, D, dtype=dtype))
    self.cmp_w1, self.cmp_b1 = mk(ch, self.cmp_len * D), nn.Parameter(torch.zeros(ch, dtype=dtype))
    self.cmp_w2, self.cmp_b2 = mk(D, ch), nn.Parameter(torch.zeros(D, dtype=dtype))
    gh = int(o.get("gate_hidden", max(8, cfg.dim // 4)))
    self.gate_w1, self.gate_b1 = mk(gh, cfg.dim), nn.Parameter(torch.zeros(gh, dtype=dtype))
    self.gate_w2, self.gate_b2 = mk(3, gh), nn.Parameter(torch.zeros(3, dtype=dtype))

  def init_weights(self, init_std: float = 0.02) -> None:
    for w in (self.qkv_w, self.cmp_w1, self.cmp_w2, self.gate_w1, self.gate_w2, self.cmp_pos):
      trunc_normal_(w, mean=0.0, std=0.02)
    trunc_normal_(self.out_w, mean=0.0, std=init_std)
    for b in (self.qkv_b, self.out_b, self.sinks, self.cmp_b1, self.cmp_b2, self.gate_b1):
      nn.init.zeros_(b)
    with torch.no_grad():   # start close to pure sliding-window attention: sigmoid -> (0.1, 0.1, 0.8)
      self.gate_b2.copy_(torch.tensor([-2.2, -2.2, 1.4], dtype=self.gate_b2.dtype))

  # ------------------------------------------------------------------ paths
  def compress(self, x: torch.Tensor) -> torch.Tensor:
    """[B,T,KV,D] -> [B,Tc,KV,D], Tc = (T - l) // d + 1 (0 when T < l)."""
    B, T, KV, D = x.shape
    l, d = self.cmp_len, self.cmp_stride
    if T < l:
      return x.new_zeros(B, 0, KV, D)
    blocks = x.permute(0, 2, 1, 3).unfold(2, l, d).permute(0, 2, 1, 4, 3) + self.cmp_pos   # [B,Tc,KV,l,D]
    Tc = blocks.size(1)
    h = torch.nn.functional.gelu(torch.nn.functional.linear(blocks.reshape(B * Tc * KV, l * D), self.cmp_w1, self.cmp_b1))
    return torch.nn.functional.linear(h, self.cmp_w2, self.cmp_b2).view(B, Tc, KV, D)

  def cmp_attention(self, qh: torch.Tensor, k_cmp: torch.Tensor, v_cmp: torch.Tensor, T: int):
    """Attention of the group-mean queries over compressed tokens + block scores [B,T,KV,Ns] (one kernel forward, two
    backward on a GPU: ops/nsa.py; the same statement in PyTorch otherwise)."""
    from ...ops.nsa import cmp_attention
    return cmp_attention(qh, k_cmp, v_cmp, cmp_len=self.cmp_len, cmp_stride=self.cmp_stride, slc_block=self.slc_block,
                         scale=self.softmax_scale)

  @torch.no_grad()
  def select_blocks(self, block_scores: torch.Tensor, T: int) -> torch.Tensor:
    """[B,T,KV,Ns] -> block ids [B,T,KV,topk] (first block, two previous blocks, then top dynamic ones)."""
    B, _, KV, Ns = block_scores.shape
    lp = self.slc_block
    t = torch.arange(T, device=block_scores.device)
    cur = t // lp
    fixed = torch.stack((torch.zeros_like(cur), (cur - 2).clamp(min=0), (cur - 1).clamp(min=0)), -1)
    fixed = fixed.view(1, T, 1, 3).expand(B, T, KV, 3)
    agg = block_scores.sum(2, keepdim=True).expand_as(block_scores).clone()
    agg = agg.masked_fill((torch.arange(Ns, device=t.device)[None, :] >= cur[:, None]).view(1, T, 1, Ns), float("-inf"))
    kd = min(max(self.topk - 3, 0), Ns)
    dyn = agg.topk(kd, dim=-1).indices if kd > 0 else fixed[..., :0]
    blocks = torch.cat((fixed, dyn), -1)
    if blocks.size(-1) < self.topk:
      blocks = torch.cat((blocks, blocks.new_zeros(B, T, KV, self.topk - blocks.size(-1))), -1)
    return blocks[..., :self.topk]

  def slc_attention(self, q, k, v, blocks: torch.Tensor) -> torch.Tensor:
    """Attention over the query's own block and its selected blocks.  On a GPU every KV group runs the tcgen05
    attention kernel with a packed bit mask built from the block list (no [T, T] tensor); the statement below it is
    the oracle for CPU tensors and unsupported head sizes."""
    B, T, H, D = q.shape
    lp = self.slc_block
    if q.is_cuda and q.dtype == torch.bfloat16 and D in (64, 128):
      cur = (torch.arange(T, device=q.device) // lp).view(1, T, 1, 1).expand(B, T, self.n_kv_heads, 1)
      with_own = torch.cat((blocks.to(torch.int32), cur.to(torch.int32)), -1)          # [B,T,KV,topk+1]
      outs = []
      for g in range(self.n_kv_heads):
        mask = SparseMask.from_blocks(with_own[:, :, g].contiguous(), lp, T)
        outs.append(attention(q[:, :, g * self.G:(g + 1) * self.G].contiguous(), k[:, :, g:g + 1].contiguous(),
                              v[:, :, g:g + 1].contiguous(), self.softmax_scale, mask=mask))
      return torch.cat(outs, dim=2)
    nb = (T + lp - 1) // lp
    allowed_blk = torch.zeros(B, T, self.n_kv_heads, nb, dtype=torch.bool, device=q.device)
    allowed_blk.scatter_(3, blocks.clamp(0, nb - 1).long(), True)
    tq = torch.arange(T, device=q.device)
    own = (tq[:, None] // lp) == (tq[None, :] // lp)
    tok = allowed_blk.permute(0, 2, 1, 3)[..., tq // lp]                     # [B,KV,T,T] by key block
    mask = (tok | own.view(1, 1, T, T)) & (tq[None, :] <= tq[:, None]).view(1, 1, T, T)
    return masked_attention(q, k, v, mask.repeat_interleave(self.G, dim=1), self.softmax_scale)

  def forward(self, x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    B, T, _ = x.shape
    H, KV, D, G = self.n_heads, self.n_kv_heads, self.head_dim, self.G
    qkv = ops.linear(x, self.qkv_w, self.qkv_b)
    q, k, v = torch.split(qkv, [H * D, KV * D, KV * D], dim=-1)
    q = ops.rope(q.reshape(B, T, H, D), cos, sin, offset=D - cos.size(-1) * 2)
    k = ops.rope(k.reshape(B, T, KV, D), cos, sin, offset=D - cos.size(-1) * 2)
    v = v.reshape(B, T, KV, D)
    qh = q.view(B, T, KV, G, D).float().mean(3).to(q.dtype)
    o_cmp, scores = self.cmp_attention(qh, self.compress(k), self.compress(v), T)
    o_slc = self.slc_attention(q, k, v, self.select_blocks(scores, T))
    o_cmp = o_cmp.unsqueeze(3).expand(B, T, KV, G, D).reshape(B, T, H, D)
    if self.window > 0:
      o_swa = attention(q, k, v, self.softmax_scale, causal=True, window=int(self.window), sinks=self.sinks)
    else:
      o_swa = torch.zeros_like(o_cmp)
    gates = torch.sigmoid(torch.nn.functional.linear(
      torch.nn.functional.gelu(torch.nn.functional.linear(x, self.gate_w1, self.gate_b1)), self.gate_w2, self.gate_b2))
    g = gates.view(B, T, 1, 3)
    o = g[..., 0:1] * o_cmp + g[..., 1:2] * o_slc + g[..., 2:3] * o_swa
    return ops.linear(o.reshape(B, T, H * D).to(x.dtype), self.out_w, self.out_b)
