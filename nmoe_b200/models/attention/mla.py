"""Multi-head Latent Attention (DeepSeek-style low-rank q / kv projections, decoupled rotary part).

Shapes follow nmoe/attention/mla.py:150-197: q = wq_b(norm(wq_a x)) split into 128 nope + 64 rope
dims per head; kv = wkv_a x split into a 512-d latent (normed, expanded by wkv_b into per-head
k_nope and v) and one shared 64-d rotary key; softmax scale (nope+rope)^-0.5; output through wo.
"""
import torch
from ..init import trunc_normal_
from torch import nn

from ... import ops
from ...ops.attention import attention, mla_attention
from ..norm import RMSNorm


class MLA(nn.Module):
  def __init__(self, cfg, dtype: torch.dtype = torch.bfloat16):
    super().__init__()
    self.dim, self.n_heads = cfg.dim, cfg.n_heads
    self.q_lora_rank, self.kv_lora_rank = cfg.q_lora_rank, cfg.kv_lora_rank
    self.nope, self.rope_dim, self.v_dim = cfg.qk_nope_head_dim, cfg.qk_rope_head_dim, cfg.v_head_dim
    self.qk_dim = self.nope + self.rope_dim
    mk = lambda o, i: nn.Parameter(torch.empty(o, i, dtype=dtype))
    self.wq_a = mk(self.q_lora_rank, self.dim)
    self.q_norm = RMSNorm(self.q_lora_rank, cfg.rms_norm_eps, dtype)
    self.wq_b = mk(self.n_heads * self.qk_dim, self.q_lora_rank)
    self.wkv_a = mk(self.kv_lora_rank + self.rope_dim, self.dim)
    self.kv_norm = RMSNorm(self.kv_lora_rank, cfg.rms_norm_eps, dtype)
    self.wkv_b = mk(self.n_heads * (self.nope + self.v_dim), self.kv_lora_rank)
    self.wo = mk(self.dim, self.n_heads * self.v_dim)
    self.softmax_scale = self.qk_dim ** -0.5
    self.window = 0

  def init_weights(self, init_std: float = 0.02) -> None:
    for w in (self.wq_a, self.wq_b, self.wkv_a, self.wkv_b):
      trunc_normal_(w, mean=0.0, std=0.02)
    trunc_normal_(self.wo, mean=0.0, std=init_std)
    self.q_norm.weight.data.fill_(1.0)
    self.kv_norm.weight.data.fill_(1.0)

  def forward(self, x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    B, S, _ = x.shape
    h = self.n_heads
    q = ops.linear(self.q_norm(ops.linear(x, self.wq_a)), self.wq_b).view(B, S, h, self.qk_dim)
    q = ops.rope(q, cos, sin, offset=self.nope)
    kv_a = ops.linear(x, self.wkv_a)
    kv_lat, k_pe = torch.split(kv_a, [self.kv_lora_rank, self.rope_dim], dim=-1)
    k_pe = ops.rope(k_pe.reshape(B, S, 1, self.rope_dim), cos, sin)
    kv = ops.linear(self.kv_norm(kv_lat.contiguous()), self.wkv_b).view(B, S, h, self.nope + self.v_dim)
    if self.window == 0:
      o = mla_attention(q, kv, k_pe, self.softmax_scale, self.nope, self.v_dim)
    else:
      k_nope, v = torch.split(kv, [self.nope, self.v_dim], dim=-1)
      k = torch.cat((k_nope, k_pe.expand(B, S, h, self.rope_dim)), dim=-1)
      o = attention(q, k, v.contiguous(), self.softmax_scale, causal=True, window=self.window)
    return ops.linear(o.reshape(B, S, h * self.v_dim), self.wo)
