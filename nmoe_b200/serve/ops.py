"""Device ops of the serving engine: paged KV store / decode attention (``csrc/paged_attention.cu``)
with plain-PyTorch statements of the same maths for CPU tensors and as test oracles."""
from __future__ import annotations

from typing import Optional

import torch

from ..ops import _lib as L


def kv_store(k: torch.Tensor, v: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, slots: torch.Tensor) -> None:
  """k, v: [N, Hkv, D] (views into a fused projection are fine: only the last two dims must be dense);
  caches: [num_blocks, block_size, Hkv, D]; slots: [N] int32, negative = skip."""
  N, Hkv, D = k.shape
  if not k.is_cuda:
    ok = slots >= 0
    kc = k_cache.view(-1, Hkv, D)
    vc = v_cache.view(-1, Hkv, D)
    kc[slots[ok].long()] = k[ok]
    vc[slots[ok].long()] = v[ok]
    return
  assert k.stride(2) == 1 and k.stride(1) == D and v.stride(2) == 1 and v.stride(1) == D
  assert k_cache.is_contiguous() and v_cache.is_contiguous() and slots.dtype == torch.int32
  L.check(L.lib().nmoe_kv_store(L.ptr(k), L.ptr(v), L.ptr(k_cache), L.ptr(v_cache), L.ptr(slots), N, Hkv * D,
                                L.c_ll(k.stride(0)), L.c_ll(v.stride(0)), L.stream()), "kv_store")


def paged_decode_reference(q, k_cache, v_cache, block_tables, context_lens, sinks, scale, window=0):
  """fp32 oracle: q [B,Hq,D] against the cached context of each sequence."""
  B, Hq, D = q.shape
  nb, bs, Hkv, _ = k_cache.shape
  g = Hq // Hkv
  out = torch.zeros(B, Hq, D, dtype=torch.float32)
  for b in range(B):
    ctx = int(context_lens[b])
    start = max(0, ctx - window) if window > 0 else 0
    pos = torch.arange(start, ctx)
    slot = block_tables[b, pos // bs].long() * bs + pos % bs
    k = k_cache.view(-1, Hkv, D)[slot].float().cpu().repeat_interleave(g, dim=1)      # [n, Hq, D]
    v = v_cache.view(-1, Hkv, D)[slot].float().cpu().repeat_interleave(g, dim=1)
    s = torch.einsum("hd,nhd->hn", q[b].float().cpu(), k) * scale
    if sinks is not None:
      s = torch.cat((s, sinks.float().cpu().view(Hq, 1)), dim=1)
    p = torch.softmax(s, dim=-1)
    if sinks is not None:
      p = p[:, :-1]
    out[b] = torch.einsum("hn,nhd->hd", p, v)
  return out


def paged_decode(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_tables: torch.Tensor,
                 context_lens: torch.Tensor, sinks: Optional[torch.Tensor], scale: float, window: int = 0) -> torch.Tensor:
  """One new token per sequence: q [B,Hq,D] -> [B,Hq,D].  ``context_lens`` counts the current token,
  whose K/V must already be in the cache."""
  if not q.is_cuda:
    return paged_decode_reference(q, k_cache, v_cache, block_tables, context_lens, sinks, scale, window).to(q.dtype)
  B, Hq, D = q.shape
  _, bs, Hkv, _ = k_cache.shape
  q = q.contiguous()
  out = torch.empty_like(q)
  sk = sinks.detach().float().contiguous() if sinks is not None else None
  assert block_tables.dtype == torch.int32 and context_lens.dtype == torch.int32 and block_tables.is_contiguous()
  L.check(L.lib().nmoe_paged_decode(L.ptr(q), L.ptr(k_cache), L.ptr(v_cache), L.ptr(block_tables), L.ptr(context_lens),
                                    L.ptr(sk), L.ptr(out), B, Hq, Hkv, D, bs, block_tables.size(1), int(window),
                                    L.c_float(scale), L.stream()), "paged_decode")
  return out
