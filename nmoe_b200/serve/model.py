"""The grading / rephrasing model of the curation stack: a gpt-oss-shaped decoder (GQA attention
with learned sinks, sliding window on even layers, YaRN rotary; top-k MoE MLP with biases and a
clamped SwiGLU) with the two execution modes a serving engine needs:

  prefill   whole (padded) prompts, K/V written to the paged cache as they are produced
  decode    one token per running sequence, attention over the paged cache

and hidden-state taps for the probe / judge heads (``return_hidden_states`` / ``up_to_layer`` /
``from_layer``: early exit and resume between layers).

CUDA path: dense projections and prefill attention on the tcgen05 kernels of this package, decode
attention and the cache scatter in ``csrc/paged_attention.cu``, experts on the block-scaled
grouped GEMM (tokens are placed and quantised to MXFP8 by the RDEP placement kernel; expert
weights ship as MXFP4 in the checkpoint and are widened once, exactly, to E4M3 with the same E8M0
scales).  CPU tensors run the same maths in plain PyTorch.

Architecture counterpart: nmoe/data/model.py:335-635 of the reference.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch
import torch.nn as nn

from .. import ops
from ..ops.attention import attention_forward
from . import ops as sops


@dataclass
class ServeConfig:
  num_hidden_layers: int = 24
  num_experts: int = 32
  experts_per_token: int = 4
  vocab_size: int = 201088
  hidden_size: int = 2880
  intermediate_size: int = 2880
  swiglu_limit: float = 7.0
  head_dim: int = 64
  num_attention_heads: int = 64
  num_key_value_heads: int = 8
  sliding_window: int = 128
  initial_context_length: int = 4096
  rope_theta: float = 150000.0
  rope_scaling_factor: float = 32.0
  rope_ntk_alpha: float = 1.0
  rope_ntk_beta: float = 32.0
  rms_eps: float = 1e-5
  probe_layer: int = 18          # hidden state after this many blocks feeds the probe head
  judge_layer: int = 24          # ... and the judge head


def yarn_inv_freq(cfg: ServeConfig, device=None) -> Tuple[torch.Tensor, float]:
  """NTK-by-parts frequencies and the attention concentration factor (YaRN)."""
  d = cfg.head_dim
  freq = cfg.rope_theta ** (torch.arange(0, d, 2, dtype=torch.float32, device=device) / d)
  if cfg.rope_scaling_factor <= 1.0:
    return 1.0 / freq, 1.0
  conc = 0.1 * math.log(cfg.rope_scaling_factor) + 1.0
  half = d / 2
  lo = half * math.log(cfg.initial_context_length / (cfg.rope_ntk_beta * 2 * math.pi)) / math.log(cfg.rope_theta)
  hi = half * math.log(cfg.initial_context_length / (cfg.rope_ntk_alpha * 2 * math.pi)) / math.log(cfg.rope_theta)
  ramp = ((torch.arange(half, dtype=torch.float32, device=device) - lo) / max(hi - lo, 1e-6)).clamp(0, 1)
  mask = 1 - ramp
  inv = (1.0 / (cfg.rope_scaling_factor * freq)) * (1 - mask) + (1.0 / freq) * mask
  return inv, conc


def apply_rotary(x: torch.Tensor, pos: torch.Tensor, inv_freq: torch.Tensor, conc: float) -> torch.Tensor:
  """x [..., H, D] with positions broadcastable to x.shape[:-2]; halves convention (x1 | x2)."""
  ang = pos.unsqueeze(-1).float() * inv_freq
  cos, sin = (ang.cos() * conc).unsqueeze(-2), (ang.sin() * conc).unsqueeze(-2)
  x1, x2 = x.float().chunk(2, dim=-1)
  return torch.cat((x1 * cos - x2 * sin, x2 * cos + x1 * sin), dim=-1).to(x.dtype)


def clamped_swiglu(h: torch.Tensor, limit: float, alpha: float = 1.702) -> torch.Tensor:
  """h [..., 2I] interleaved (gate even, linear odd) -> [..., I]."""
  g, u = h[..., ::2].float(), h[..., 1::2].float()
  g = g.clamp(max=limit)
  u = u.clamp(-limit, limit)
  return (g * torch.sigmoid(alpha * g) * (u + 1)).to(h.dtype)


class CacheView:
  """What a forward pass needs to know about the paged cache for one step."""

  def __init__(self, k_cache, v_cache, slots, *, block_tables=None, context_lens=None, prefix_lens=None, block_size=16):
    self.k_cache, self.v_cache = k_cache, v_cache          # [L, num_blocks, block_size, Hkv, D]
    self.slots = slots                                      # prefill: [B, S] int32 (-1 = padding), decode: [B]
    self.block_tables, self.context_lens = block_tables, context_lens
    self.prefix_lens = prefix_lens                          # prefill: cached tokens per sequence (host list) or None
    self.block_size = block_size


class Attention(nn.Module):
  def __init__(self, cfg: ServeConfig, layer: int, dtype):
    super().__init__()
    self.cfg, self.layer = cfg, layer
    self.nq, self.nkv, self.d = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    self.window = cfg.sliding_window if layer % 2 == 0 else 0
    self.scale = 1.0 / math.sqrt(cfg.head_dim)
    self.norm = nn.Parameter(torch.ones(cfg.hidden_size, dtype=dtype))
    self.qkv_w = nn.Parameter(torch.empty(self.d * (self.nq + 2 * self.nkv), cfg.hidden_size, dtype=dtype))
    self.qkv_b = nn.Parameter(torch.zeros(self.d * (self.nq + 2 * self.nkv), dtype=dtype))
    self.out_w = nn.Parameter(torch.empty(cfg.hidden_size, self.d * self.nq, dtype=dtype))
    self.out_b = nn.Parameter(torch.zeros(cfg.hidden_size, dtype=dtype))
    self.sinks = nn.Parameter(torch.zeros(self.nq, dtype=dtype))

  def _qkv(self, x, pos, rot):
    qkv = ops.linear(ops.rmsnorm(x, self.norm, self.cfg.rms_eps), self.qkv_w, self.qkv_b)
    lead = x.shape[:-1]
    q, k, v = qkv.split([self.nq * self.d, self.nkv * self.d, self.nkv * self.d], dim=-1)
    q = apply_rotary(q.reshape(*lead, self.nq, self.d), pos, *rot)
    k = apply_rotary(k.reshape(*lead, self.nkv, self.d), pos, *rot)
    return q, k, v.reshape(*lead, self.nkv, self.d)

  def prefill(self, x, pos, rot, cache: Optional[CacheView]):
    """x [B,S,H]; positions [B,S] (absolute).  Sequences with a cached prefix attend to it through
    keys/values gathered from the cache (their own rows are written first)."""
    B, S, _ = x.shape
    q, k, v = self._qkv(x, pos, rot)
    if cache is not None:
      sops.kv_store(k.reshape(B * S, self.nkv, self.d).contiguous(), v.reshape(B * S, self.nkv, self.d).contiguous(),
                    cache.k_cache[self.layer], cache.v_cache[self.layer], cache.slots.reshape(-1))
    has_prefix = cache is not None and cache.prefix_lens is not None and any(p > 0 for p in cache.prefix_lens)
    if not has_prefix:
      o = self._dense_attention(q, k, v)
    else:
      o = torch.empty(B, S, self.nq, self.d, dtype=x.dtype, device=x.device)
      for b in range(B):
        p = int(cache.prefix_lens[b])
        if p == 0:
          o[b:b + 1] = self._dense_attention(q[b:b + 1], k[b:b + 1], v[b:b + 1])
          continue
        n = int((cache.slots[b] >= 0).sum())                  # new tokens of this sequence
        tab = cache.block_tables[b].long()
        idx = torch.arange(p, device=x.device)
        slot = tab[idx // cache.block_size] * cache.block_size + idx % cache.block_size
        kc = cache.k_cache[self.layer].view(-1, self.nkv, self.d)[slot]
        vc = cache.v_cache[self.layer].view(-1, self.nkv, self.d)[slot]
        qf = torch.cat((torch.zeros(p, self.nq, self.d, dtype=x.dtype, device=x.device), q[b, :n]), 0).unsqueeze(0)
        kf = torch.cat((kc, k[b, :n]), 0).unsqueeze(0)
        vf = torch.cat((vc, v[b, :n]), 0).unsqueeze(0)
        o[b, :n] = self._dense_attention(qf, kf, vf)[0, p:]
        o[b, n:] = 0
    return x + ops.linear(o.reshape(B, S, self.nq * self.d), self.out_w, self.out_b)

  def _dense_attention(self, q, k, v):
    if q.is_cuda:
      return attention_forward(q, k, v, self.scale, self.window, self.sinks, need_lse=False)[0]
    return ops.attention(q, k, v, self.scale, window=self.window, sinks=self.sinks)

  def decode(self, x, pos, rot, cache: CacheView):
    """x [B,H]: one token per sequence."""
    q, k, v = self._qkv(x, pos, rot)
    sops.kv_store(k.contiguous(), v.contiguous(), cache.k_cache[self.layer], cache.v_cache[self.layer], cache.slots)
    o = sops.paged_decode(q, cache.k_cache[self.layer], cache.v_cache[self.layer], cache.block_tables,
                          cache.context_lens, self.sinks, self.scale, self.window)
    return x + ops.linear(o.reshape(x.size(0), self.nq * self.d), self.out_w, self.out_b)


class MoEMLP(nn.Module):
  """Top-k routed MLP with biases: softmax over the selected logits, clamped SwiGLU."""

  def __init__(self, cfg: ServeConfig, dtype):
    super().__init__()
    self.cfg = cfg
    E, H, I = cfg.num_experts, cfg.hidden_size, cfg.intermediate_size
    self.norm = nn.Parameter(torch.ones(H, dtype=dtype))
    self.gate_w = nn.Parameter(torch.empty(E, H, dtype=dtype))
    self.gate_b = nn.Parameter(torch.zeros(E, dtype=dtype))
    self.w1 = nn.Parameter(torch.empty(E, 2 * I, H, dtype=dtype))      # gate / linear rows interleaved
    self.b1 = nn.Parameter(torch.zeros(E, 2 * I, dtype=dtype))
    self.w2 = nn.Parameter(torch.empty(E, H, I, dtype=dtype))
    self.b2 = nn.Parameter(torch.zeros(E, H, dtype=dtype))
    self._q = None           # (w1q, w1sf, w2q, w2sf, n2_pad) block-scaled copies, built on first CUDA use
    self.rdep = None         # set by Transformer: shared dispatch scratch

  def _route(self, xn):
    logits = ops.linear(xn, self.gate_w, self.gate_b).float()
    val, eid = logits.topk(self.cfg.experts_per_token, dim=-1)
    return torch.softmax(val, dim=-1), eid

  def _quantised(self):
    if self._q is None:
      from ..ops import quant as Q
      def pack(w):
        # scale atoms cover 128 output rows: pad every expert's row count to a multiple of 128 with zero rows
        E, n, k = w.shape
        n_pad = (n + 127) // 128 * 128
        if n_pad != n:
          w = torch.cat((w, w.new_zeros(E, n_pad - n, k)), dim=1)
        q, sf = Q.quant_mxfp8(w.reshape(E * n_pad, k))
        return q.view(E, n_pad, k), sf
      w1q, w1sf = pack(self.w1.detach())
      w2q, w2sf = pack(self.w2.detach())
      self._q = (w1q, w1sf, w2q, w2sf)
    return self._q

  def forward(self, x: torch.Tensor) -> torch.Tensor:
    shape = x.shape
    X = x.reshape(-1, shape[-1])
    xn = ops.rmsnorm(X, self.norm, self.cfg.rms_eps)
    gates, eid = self._route(xn)
    if not X.is_cuda or self.rdep is None:
      out = torch.zeros_like(X, dtype=torch.float32)
      for e in eid.unique().tolist():
        tok, slot = (eid == e).nonzero(as_tuple=True)
        h = xn[tok].float() @ self.w1[e].float().t() + self.b1[e].float()
        a = clamped_swiglu(h, self.cfg.swiglu_limit)
        y = a @ self.w2[e].float().t() + self.b2[e].float()
        out.index_add_(0, tok, y * gates[tok, slot].unsqueeze(-1))
      return x + out.to(x.dtype).view(shape)
    from ..ops import quant as Q
    rd = self.rdep
    H = X.size(1)
    w1q, w1sf, w2q, w2sf = self._quantised()
    N1 = self.w1.size(1)
    out = torch.empty_like(X)
    for t0 in range(0, X.size(0), rd.max_tokens):            # the dispatch scratch is sized for max_tokens rows
      xs, g, ei = xn[t0:t0 + rd.max_tokens].contiguous(), gates[t0:t0 + rd.max_tokens].contiguous(), eid[t0:t0 + rd.max_tokens]
      plan = rd.plan(ei.int().contiguous())
      rd.place_mx(xs, plan, g.view(-1))
      rd.wait_data()
      # the dispatch scratch is sized for max_tokens, but this call's rows (each expert's segment padded to 128) cannot
      # exceed T*K + E*127: everything below works on that prefix, so a decode step of a few sequences does not pay
      # for elementwise passes over tens of thousands of unused rows
      n_rows = min(rd.xq.size(0), (xs.size(0) * self.cfg.experts_per_token + self.cfg.num_experts * 127 + 127) // 128 * 128)
      h = Q.grouped_gemm_mxfp8(rd.xq[:n_rows], rd.sfa, w1q, w1sf, plan.tile_expert, plan.n_m_tiles)
      # rows past the valid tiles hold stale data; they are never read back (the pushes skip them)
      row_e = plan.tile_expert[:h.size(0) // 128].clamp(0, self.cfg.num_experts - 1).long().repeat_interleave(128)
      a = clamped_swiglu(torch.nan_to_num(h[:, :N1] + self.b1[row_e]), self.cfg.swiglu_limit)
      aq, asf = Q.quant_mxfp8(a, plan.n_m_tiles)
      y = Q.grouped_gemm_mxfp8(aq, asf, w2q, w2sf, plan.tile_expert, plan.n_m_tiles)
      y = (y[:, :H] + self.b2[row_e]).contiguous()
      rd.push_and_reduce(y, plan, g.float().contiguous().view(-1), None, out[t0:t0 + xs.size(0)])
    return x + out.view(shape)


class Transformer(nn.Module):
  def __init__(self, cfg: ServeConfig, *, dtype=torch.bfloat16, device=None, max_tokens: int = 8192):
    super().__init__()
    self.cfg = cfg
    with torch.device(device or "cpu"):
      self.embed = nn.Parameter(torch.empty(cfg.vocab_size, cfg.hidden_size, dtype=dtype))
      self.attn = nn.ModuleList([Attention(cfg, i, dtype) for i in range(cfg.num_hidden_layers)])
      self.mlp = nn.ModuleList([MoEMLP(cfg, dtype) for _ in range(cfg.num_hidden_layers)])
      self.norm = nn.Parameter(torch.ones(cfg.hidden_size, dtype=dtype))
      self.unembed = nn.Parameter(torch.empty(cfg.vocab_size, cfg.hidden_size, dtype=dtype))
    inv, conc = yarn_inv_freq(cfg, device)
    self.register_buffer("inv_freq", inv, persistent=False)
    self.conc = conc
    self.rdep = None
    if device is not None and torch.device(device).type == "cuda":
      from ..parallel.rdep import Rdep
      self.rdep = Rdep(cfg.hidden_size, cfg.num_experts, cfg.experts_per_token, max_tokens, device=torch.device(device),
                       profile="fp8", group=None, single_process=True)
      for m in self.mlp:
        m.rdep = self.rdep

  @torch.no_grad()
  def init_weights(self, std: float = 0.02, seed: int = 0) -> None:
    from ..models.init import normal_
    gen = torch.Generator(device=self.embed.device).manual_seed(seed)
    for name, p in self.named_parameters():
      if name.endswith(("norm", ".norm")):
        p.fill_(1.0)
      elif name.endswith(("_b", "b1", "b2")):
        p.zero_()
      elif name.endswith("sinks"):
        normal_(p, 0.0, 1.0, gen)
      else:
        normal_(p, 0.0, std, gen)

  def forward(self, input_ids: torch.Tensor, positions: torch.Tensor, *, cache: Optional[CacheView] = None,
              is_prefill: bool = True, return_hidden_states: bool = False, up_to_layer: Optional[int] = None,
              from_layer: Optional[int] = None, hidden_in: Optional[torch.Tensor] = None, no_logits: bool = False):
    """prefill: input_ids / positions [B,S]; decode: [B].  ``from_layer`` resumes from ``hidden_in``
    (the state returned by an earlier call that stopped at ``up_to_layer``).  Returns logits (fp32),
    or (logits | None, {layer: hidden}) with ``return_hidden_states``; a call that stops before the
    last layer returns its final hidden state under key ``up_to_layer``."""
    L = self.cfg.num_hidden_layers
    start = 0 if from_layer is None else max(0, min(L, int(from_layer)))
    stop = L if up_to_layer is None else max(start, min(L, int(up_to_layer)))
    x = hidden_in if (start > 0 and hidden_in is not None) else ops.embedding(input_ids, self.embed, 1.0)
    rot = (self.inv_freq, self.conc)
    taps: Dict[int, torch.Tensor] = {}
    for i in range(start, stop):
      x = self.attn[i].prefill(x, positions, rot, cache) if is_prefill else self.attn[i].decode(x, positions, rot, cache)
      x = self.mlp[i](x)
      if return_hidden_states and (i + 1) in (self.cfg.probe_layer, self.cfg.judge_layer):
        taps[i + 1] = x.detach()
    if return_hidden_states or stop < L:
      taps[stop] = x.detach()
    if stop < L:
      return None, taps
    logits = None
    if not no_logits:
      logits = ops.linear(ops.rmsnorm(x, self.norm, self.cfg.rms_eps), self.unembed).float()
    return (logits, taps) if return_hidden_states else logits


def pool_hidden(hidden: torch.Tensor, mask: Optional[torch.Tensor] = None) -> torch.Tensor:
  """Mean over the sequence dim of [B,S,H], counting only ``mask``-ed positions (nmoe/data/model.py:637-644)."""
  if mask is None:
    return hidden.float().mean(dim=1)
  m = mask.to(torch.float32)
  return (hidden.float() * m.unsqueeze(-1)).sum(1) / m.sum(1).clamp(min=1).unsqueeze(-1)
