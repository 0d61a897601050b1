"""Decoder-only MoE transformer (reference: nmoe/model.py:141-270).

embedding * 10.667 -> blocks (pre-norm attention + pre-norm FFN; the first ``n_dense_layers``
FFNs are dense SwiGLU MLPs, the rest are MoE layers) -> final RMSNorm -> lm_head * 0.125.
Global layers use ``cfg.attn``; with ``attn_global_every`` > 1 the other layers use
``cfg.attn_local`` with a sliding window.  Attention sub-blocks are recomputed in backward
(activation checkpointing) unless ``cfg.activation_checkpoint == "none"``.

``forward`` returns logits; ``loss`` goes through the fused lm_head + cross-entropy op and
never materialises the [tokens, vocab] logits.
"""
from __future__ import annotations

import os

from typing import List, Optional, Tuple

import torch
from .init import normal_, trunc_normal_
import torch.distributed as dist
from torch import nn
from torch.utils.checkpoint import checkpoint

from .. import ops
from ..config import Config
from ..parallel.rdep import Rdep
from ..utils.profiling import scope
from .attention import get_attention
from .mlp import MLP
from .moe import MoE
from .norm import RMSNorm
from .rope import RotaryEmbedding

MUP_EMBED_SCALE = 10.667
LOGIT_SCALE = 0.125


class TransformerBlock(nn.Module):
  def __init__(self, cfg: Config, layer_id: int, *, rdep: Optional[Rdep], n_local: int, dtype: torch.dtype):
    super().__init__()
    self.layer_id = layer_id
    self.attn_norm = RMSNorm(cfg.dim, cfg.rms_norm_eps, dtype)
    self.ffn_norm = RMSNorm(cfg.dim, cfg.rms_norm_eps, dtype)
    self.is_global = cfg.is_global_layer(layer_id)
    name = cfg.attn if self.is_global else cfg.attn_local
    self.attn = get_attention(name)(cfg, dtype)
    if not self.is_global:
      if not hasattr(self.attn, "window"):
        raise ValueError(f"local attention '{name}' has no 'window' attribute")
      self.attn.window = int(cfg.attn_local_window)
    self.is_moe = layer_id >= cfg.n_dense_layers
    if self.is_moe:
      self.ffn = MoE(cfg, layer_id, rdep=rdep, n_local=n_local, dtype=dtype)
    else:
      self.ffn = MLP(cfg.dim, cfg.inter_dim, dtype)
    self.init_std = 0.02 / (2 * (layer_id + 1)) ** 0.5
    self.ckpt = cfg.activation_checkpoint
    self._scope_attn = f"block_{layer_id:02d}/attn_{'global' if self.is_global else 'local'}"
    self._scope_ffn = f"block_{layer_id:02d}/{'moe' if self.is_moe else 'mlp'}"

  def init_weights(self) -> None:
    self.attn_norm.weight.data.fill_(1.0)
    self.ffn_norm.weight.data.fill_(1.0)
    self.attn.init_weights(self.init_std)
    self.ffn.init_weights(self.init_std)

  def _attn(self, x, cos, sin):
    return self.attn(self.attn_norm(x), cos, sin)

  def _ffn(self, x):
    return self.ffn(self.ffn_norm(x))

  def forward(self, x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    with scope(self._scope_attn):
      if self.ckpt != "none" and torch.is_grad_enabled():
        x = x + checkpoint(self._attn, x, cos, sin, use_reentrant=False)
      else:
        x = x + self._attn(x, cos, sin)
    with scope(self._scope_ffn):
      return x + self._ffn(x)


class Transformer(nn.Module):
  def __init__(self, cfg: Config, *, dtype: torch.dtype = torch.bfloat16, device: Optional[torch.device] = None,
               rdep: Optional[Rdep] = None, tokens_per_rank: Optional[int] = None):
    """``tokens_per_rank`` sizes the RDEP buffers (default batch_size/world * seq_len)."""
    super().__init__()
    world = dist.get_world_size() if dist.is_initialized() else 1
    cfg.validate(world)
    self.cfg = cfg
    self.world = world
    n_local = (cfg.n_routed_experts // world) if cfg.has_moe else 0
    self.n_local = n_local
    on_cuda = device is not None and torch.device(device).type == "cuda"
    if cfg.has_moe and on_cuda and rdep is None:
      tpr = tokens_per_rank or max(1, cfg.batch_size // world) * cfg.seq_len
      rdep = Rdep(cfg.dim, cfg.n_routed_experts, cfg.n_activated_experts, tpr, device=torch.device(device),
                  profile=cfg.dtype, capacity_factor=cfg.rdep_capacity_factor)
    pipe = os.environ.get("NMOE_MOE_PIPELINE", str(getattr(cfg, "moe_pipeline", "false"))).lower()
    if rdep is not None and (pipe in ("1", "true", "yes", "on")):
      rdep.make_halves()
    self.rdep = rdep
    with torch.device(device or "cpu"):
      self.embedding = nn.Parameter(torch.empty(cfg.vocab_size, cfg.dim, dtype=dtype))
      self.rope = RotaryEmbedding(cfg.qk_rope_head_dim, cfg.rope_theta, cfg.max_position_embeddings,
                                  cfg.max_position_embeddings * 2, cfg.rope_scaling_factor, cfg.rope_ntk_alpha,
                                  cfg.rope_ntk_beta)
      self.blocks = nn.ModuleList([TransformerBlock(cfg, i, rdep=rdep, n_local=n_local, dtype=dtype)
                                   for i in range(cfg.n_layers)])
      self.norm = RMSNorm(cfg.dim, cfg.rms_norm_eps, dtype)
      self.lm_head = nn.Parameter(torch.empty(cfg.vocab_size, cfg.dim, dtype=dtype))

  # ------------------------------------------------------------------ init / param sets
  @torch.no_grad()
  def init_weights(self) -> None:
    normal_(self.embedding, mean=0.0, std=0.02)
    for blk in self.blocks:
      blk.init_weights()
    self.norm.weight.data.fill_(1.0)
    trunc_normal_(self.lm_head, mean=0.0, std=self.cfg.dim ** -0.5)

  def moe_layers(self) -> List[MoE]:
    return [b.ffn for b in self.blocks if isinstance(b.ffn, MoE)]

  def param_sets(self) -> Tuple[List[nn.Parameter], List[nn.Parameter]]:
    """(expert params, everything else).  Experts are rank-local and never reduced across ranks."""
    experts: List[nn.Parameter] = []
    for m in self.moe_layers():
      experts += [m.W13, m.W2]
    ids = {id(p) for p in experts}
    return experts, [p for p in self.parameters() if id(p) not in ids]

  # ------------------------------------------------------------------ forward
  def hidden(self, tokens: torch.Tensor) -> torch.Tensor:
    with scope("embed"):
      x = ops.embedding(tokens, self.embedding, MUP_EMBED_SCALE)
    S = tokens.size(1)
    cos, sin = self.rope.cos[:S], self.rope.sin[:S]
    for m in self.moe_layers():
      m.loads.zero_()
    for blk in self.blocks:
      x = blk(x, cos, sin)
    with scope("final_norm"):
      return self.norm(x)

  def forward(self, tokens: torch.Tensor) -> torch.Tensor:
    return ops.linear(self.hidden(tokens), self.lm_head) * LOGIT_SCALE

  def loss(self, tokens: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
    """Mean CE over targets != eos_token_id (nmoe/train.py:102-105)."""
    h = self.hidden(tokens)
    with scope("lm_head_loss"):
      return ops.lm_head_loss(h.reshape(-1, h.size(-1)), self.lm_head, targets.reshape(-1), self.cfg.eos_token_id,
                              LOGIT_SCALE)

  @torch.no_grad()
  def expert_loads(self) -> Optional[torch.Tensor]:
    """[n_moe_layers, E] selection counts of the last forward, summed over ranks (fp32)."""
    layers = self.moe_layers()
    if not layers:
      return None
    loads = torch.stack([m.loads for m in layers], dim=0).float()
    if dist.is_initialized() and self.world > 1:
      dist.all_reduce(loads, op=dist.ReduceOp.SUM)
    return loads
