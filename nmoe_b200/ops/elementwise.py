"""RMSNorm, rotary, SwiGLU and embedding as autograd ops.

CUDA tensors run the kernels in ``csrc/elementwise.cu``; CPU tensors run the
fp32 oracle in ``nmoe_b200.ref.ops`` (that path is what the CPU tests exercise).
"""
from __future__ import annotations

import torch

from ..ref import ops as R
from . import _lib as L


def _scratch(device, nfloat: int) -> torch.Tensor:
  return torch.empty(nfloat, dtype=torch.float32, device=device)


# ------------------------------------------------------------------ RMSNorm
class _RMSNorm(torch.autograd.Function):
  @staticmethod
  def forward(ctx, x, w, eps):
    H = x.size(-1)
    x2 = x.contiguous().view(-1, H)
    M = x2.size(0)
    y = torch.empty_like(x2)
    rstd = torch.empty(M, dtype=torch.float32, device=x.device)
    L.check(L.lib().nmoe_rmsnorm_fwd(L.ptr(x2), L.ptr(w), L.ptr(y), L.ptr(rstd), M, H, L.c_float(eps), L.stream()),
            "rmsnorm_fwd")
    ctx.save_for_backward(x2, w, rstd)
    ctx.shape = x.shape
    return y.view(x.shape)

  @staticmethod
  def backward(ctx, dy):
    x2, w, rstd = ctx.saved_tensors
    M, H = x2.shape
    dy2 = dy.contiguous().view(M, H)
    dx = torch.empty_like(x2)
    dw = torch.empty_like(w)
    nb = L.lib().nmoe_rmsnorm_bwd_blocks(M)
    scratch = _scratch(x2.device, nb * H + M)      # partial column sums, then one row dot per row (wide rows only)
    L.check(L.lib().nmoe_rmsnorm_bwd_twopass(L.ptr(dy2), L.ptr(x2), L.ptr(w), L.ptr(rstd), L.ptr(dx), L.ptr(dw),
                                             L.ptr(scratch), M, H, 0, L.stream()), "rmsnorm_bwd", 3)
    return dx.view(ctx.shape), dw, None


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
  if x.is_cuda and x.dtype == torch.bfloat16:
    return _RMSNorm.apply(x, w, eps)
  return R.rmsnorm(x, w, eps)


# ------------------------------------------------------------------ rotary
def _rope_launch(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, offset: int, D: int, backward: bool) -> None:
  """x: [B,S,h,Dtot] with a dense last dim; rotates x[..., offset:offset+D] in place."""
  B, S, h, Dt = x.shape
  assert x.stride(-1) == 1 and x.stride(2) * h == x.stride(1) and x.stride(1) * S == x.stride(0), \
    "rope expects [B,S,h,D] rows at a uniform stride"
  L.check(L.lib().nmoe_rope_inplace(L.ptr(x), L.ptr(cos), L.ptr(sin), L.c_ll(B * S * h), h, S,
                                    L.c_ll(x.stride(2)), offset, D, int(backward), L.stream()), "rope")


class _Rope(torch.autograd.Function):
  """Out-of-place for autograd's sake (one copy), rotating the trailing D dims of each head."""

  @staticmethod
  def forward(ctx, x, cos, sin, offset, D):
    y = x.contiguous().clone()
    _rope_launch(y, cos, sin, offset, D, False)
    ctx.save_for_backward(cos, sin)
    ctx.offset, ctx.D = offset, D
    return y

  @staticmethod
  def backward(ctx, dy):
    cos, sin = ctx.saved_tensors
    dx = dy.contiguous().clone()
    _rope_launch(dx, cos, sin, ctx.offset, ctx.D, True)
    return dx, None, None, None, None


def rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, offset: int = 0) -> torch.Tensor:
  """Rotate x[..., offset:] (x: [B,S,h,Dtot]); cos/sin: fp32 [>=S, (Dtot-offset)/2]."""
  D = x.size(-1) - offset
  if x.is_cuda and x.dtype == torch.bfloat16:
    return _Rope.apply(x, cos.float().contiguous(), sin.float().contiguous(), offset, D)
  if offset == 0:
    return R.rope(x, cos, sin)
  return torch.cat((x[..., :offset], R.rope(x[..., offset:], cos, sin)), dim=-1)


# ------------------------------------------------------------------ SwiGLU (interleaved gate/up)
class _SwiGLU(torch.autograd.Function):
  @staticmethod
  def forward(ctx, h13):
    F2 = h13.size(-1)
    h = h13.contiguous().view(-1, F2)
    a = torch.empty(h.size(0), F2 // 2, dtype=h.dtype, device=h.device)
    L.check(L.lib().nmoe_swiglu_fwd(L.ptr(h), L.ptr(a), L.c_ll(h.size(0)), F2 // 2, None, L.stream()), "swiglu_fwd")
    ctx.save_for_backward(h)
    ctx.shape = h13.shape
    return a.view(*h13.shape[:-1], F2 // 2)

  @staticmethod
  def backward(ctx, da):
    (h,) = ctx.saved_tensors
    M, F2 = h.shape
    d = da.contiguous().view(M, F2 // 2)
    dh = torch.empty_like(h)
    L.check(L.lib().nmoe_swiglu_bwd(L.ptr(h), L.ptr(d), L.ptr(dh), None, None, None, L.c_ll(M), F2 // 2, None, L.stream()),
            "swiglu_bwd")
    return dh.view(ctx.shape)


def swiglu(h13: torch.Tensor) -> torch.Tensor:
  """h13[..., 2F] with gate at even and up at odd columns -> silu(gate) * up  [..., F]."""
  if h13.is_cuda and h13.dtype == torch.bfloat16:
    return _SwiGLU.apply(h13)
  return R.swiglu(h13[..., 0::2], h13[..., 1::2])


def swiglu_rows(h13: torch.Tensor, n_tiles: torch.Tensor | None = None) -> torch.Tensor:
  """No-autograd SwiGLU over [M,2F]; with ``n_tiles`` (device int32[1]) only rows < n_tiles*128 are computed."""
  M, F2 = h13.shape
  if h13.is_cuda:
    a = torch.empty(M, F2 // 2, dtype=h13.dtype, device=h13.device)
    L.check(L.lib().nmoe_swiglu_fwd(L.ptr(h13), L.ptr(a), L.c_ll(M), F2 // 2, L.ptr(n_tiles), L.stream()), "swiglu_fwd")
    return a
  return R.swiglu(h13[:, 0::2], h13[:, 1::2])


def swiglu_bwd_fused(h13: torch.Tensor, da: torch.Tensor, row_scale: torch.Tensor | None, want_rowdot: bool,
                     want_a: bool, n_tiles: torch.Tensor | None = None):
  """MoE backward helper: returns (dh13, rowdot or None, a*scale or None).

  dh13 is the gradient of swiglu at h13 for upstream ``da * row_scale``; rowdot[m] =
  <swiglu(h13)[m], da[m]> (the routing-gate gradient); a_out = swiglu(h13) * row_scale.
  """
  M, F2 = h13.shape
  if h13.is_cuda:
    dh = torch.empty_like(h13)
    rd = torch.empty(M, dtype=torch.float32, device=h13.device) if want_rowdot else None
    ao = torch.empty(M, F2 // 2, dtype=h13.dtype, device=h13.device) if want_a else None
    L.check(L.lib().nmoe_swiglu_bwd(L.ptr(h13), L.ptr(da), L.ptr(dh), L.ptr(row_scale), L.ptr(rd), L.ptr(ao),
                                    L.c_ll(M), F2 // 2, L.ptr(n_tiles), L.stream()), "swiglu_bwd")
    return dh, rd, ao
  g, u = h13[:, 0::2].float(), h13[:, 1::2].float()
  s = torch.sigmoid(g)
  a = g * s * u
  sc = row_scale.float().unsqueeze(-1) if row_scale is not None else 1.0
  d = da.float() * sc
  dh = torch.empty_like(h13, dtype=torch.float32)
  dh[:, 0::2] = d * u * s * (1 + g * (1 - s))
  dh[:, 1::2] = d * g * s
  rd = (a * da.float()).sum(-1) if want_rowdot else None
  return dh.to(h13.dtype), rd, ((a * sc).to(h13.dtype) if want_a else None)


# ------------------------------------------------------------------ embedding
class _Embedding(torch.autograd.Function):
  @staticmethod
  def forward(ctx, tokens, table, scale):
    T = tokens.numel()
    V, H = table.shape
    out = torch.empty(T, H, dtype=table.dtype, device=table.device)
    tk = tokens.contiguous().view(-1).long()
    L.check(L.lib().nmoe_embedding_fwd(L.ptr(tk), L.ptr(table), L.ptr(out), L.c_ll(T), H, V, L.c_float(scale),
                                       L.stream()), "embedding_fwd")
    ctx.save_for_backward(tk)
    ctx.V, ctx.scale = V, scale
    return out.view(*tokens.shape, H)

  @staticmethod
  def backward(ctx, dout):
    (tk,) = ctx.saved_tensors
    H = dout.size(-1)
    dtab = torch.zeros(ctx.V, H, dtype=dout.dtype, device=dout.device)
    dtab.index_add_(0, tk, dout.reshape(-1, H), alpha=ctx.scale)
    return None, dtab, None


def embedding(tokens: torch.Tensor, table: torch.Tensor, scale: float) -> torch.Tensor:
  if table.is_cuda and table.dtype == torch.bfloat16:
    return _Embedding.apply(tokens, table, scale)
  return torch.nn.functional.embedding(tokens, table) * scale
