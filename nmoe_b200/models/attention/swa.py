"""Sliding-window attention with fused QKV (+bias), GQA and learned per-head sinks
(nmoe/attention/swa.py:10-85): head_dim = v_head_dim, rotary on the trailing qk_rope_head_dim
dims, the sink logit enters the softmax denominator only, window = ``self.window`` (0 = full causal).
"""
import torch
from ..init import trunc_normal_
from torch import nn

from ... import ops
from ...ops.attention import attention


class SWA(nn.Module):
  def __init__(self, cfg, dtype: torch.dtype = torch.bfloat16):
    super().__init__()
    self.dim, self.n_heads = cfg.dim, cfg.n_heads
    self.head_dim = int(cfg.v_head_dim)
    self.rope_dim = int(cfg.qk_rope_head_dim)
    if not (0 <= self.rope_dim <= self.head_dim) or self.rope_dim % 2:
      raise ValueError(f"SWA needs an even qk_rope_head_dim in [0, v_head_dim]; got {self.rope_dim}/{self.head_dim}")
    self.nope = self.head_dim - self.rope_dim
    self.n_kv_heads = int((cfg.attn_swa or {}).get("kv_heads", self.n_heads))
    if self.n_heads % self.n_kv_heads:
      raise ValueError(f"n_heads ({self.n_heads}) must be a multiple of kv_heads ({self.n_kv_heads})")
    out_feats = (self.n_heads + 2 * self.n_kv_heads) * self.head_dim
    self.qkv_w = nn.Parameter(torch.empty(out_feats, self.dim, dtype=dtype))
    self.qkv_b = nn.Parameter(torch.zeros(out_feats, dtype=dtype))
    self.out_w = nn.Parameter(torch.empty(self.dim, self.n_heads * self.head_dim, dtype=dtype))
    self.out_b = nn.Parameter(torch.zeros(self.dim, dtype=dtype))
    self.sinks = nn.Parameter(torch.zeros(self.n_heads, dtype=dtype))
    self.window = 0
    self.softmax_scale = self.head_dim ** -0.5

  def init_weights(self, init_std: float = 0.02) -> None:
    trunc_normal_(self.qkv_w, mean=0.0, std=0.02)
    trunc_normal_(self.out_w, mean=0.0, std=init_std)
    for p in (self.qkv_b, self.out_b, self.sinks):
      nn.init.zeros_(p)

  def forward(self, x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    B, S, _ = x.shape
    H, KV, D = self.n_heads, self.n_kv_heads, self.head_dim
    qkv = ops.linear(x, self.qkv_w, self.qkv_b)
    q, k, v = torch.split(qkv, [H * D, KV * D, KV * D], dim=-1)
    q = q.reshape(B, S, H, D)
    k = k.reshape(B, S, KV, D)
    v = v.reshape(B, S, KV, D)
    if self.rope_dim:
      q = ops.rope(q, cos, sin, offset=self.nope)
      k = ops.rope(k, cos, sin, offset=self.nope)
    o = attention(q, k, v, self.softmax_scale, causal=True, window=int(self.window), sinks=self.sinks)
    return ops.linear(o.reshape(B, S, H * D), self.out_w, self.out_b)
