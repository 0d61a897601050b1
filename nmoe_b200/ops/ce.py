"""lm_head + masked cross-entropy without materialising [T, V] logits.

Token rows are processed in chunks: logits chunk = h_c @ W^T (tcgen05 GEMM), the CE kernel turns
the chunk into its gradient in place while accumulating the loss, and the two backward GEMMs
(dh_c, dW +=) run right away.  The autograd backward only scales the stored gradients.
"""
from __future__ import annotations

import torch

from ..ref import ops as R
from . import _lib as L
from . import tc_gemm as G


class _LMHeadLoss(torch.autograd.Function):
  @staticmethod
  def forward(ctx, h, w, targets, ignore_id, logit_scale, chunk_rows):
    T, H = h.shape
    V = w.size(0)
    dev = h.device
    tg = targets.reshape(-1).long().contiguous()
    inv_count = 1.0 / (tg != ignore_id).sum().clamp(min=1).float()
    inv_count = inv_count.reshape(1).contiguous()
    loss = torch.zeros(1, dtype=torch.float32, device=dev)
    need_grad = ctx.needs_input_grad[0] or ctx.needs_input_grad[1]
    dh = torch.empty_like(h) if need_grad else None
    dw32 = torch.zeros(V, H, dtype=torch.float32, device=dev) if need_grad else None
    for r0 in range(0, T, chunk_rows):
      r1 = min(T, r0 + chunk_rows)
      hc = h[r0:r1]
      logits = G.gemm(hc, w)
      L.check(L.lib().nmoe_ce_fwd_bwd(L.ptr(logits), L.ptr(tg[r0:r1]), r1 - r0, V, L.c_ll(logits.stride(0)),
                                      int(ignore_id), L.c_float(logit_scale), L.ptr(inv_count), L.ptr(loss), None,
                                      int(need_grad), L.stream()), "ce_fwd_bwd")
      if need_grad:
        G.gemm(logits, w, b_mn=True, out=dh[r0:r1])
        G.gemm(logits, hc, a_mn=True, b_mn=True, out=dw32, accumulate=True)
      del logits
    if need_grad:
      ctx.save_for_backward(dh, dw32.to(w.dtype))
    return loss.squeeze(0)

  @staticmethod
  def backward(ctx, g):
    dh, dw = ctx.saved_tensors
    return dh * g.to(dh.dtype), dw * g.to(dw.dtype), None, None, None, None


def lm_head_loss(h: torch.Tensor, w: torch.Tensor, targets: torch.Tensor, ignore_id: int, logit_scale: float,
                 chunk_rows: int = 4096) -> torch.Tensor:
  """Mean over unmasked positions of CE((h @ w^T) * logit_scale, targets); h [T,H], w [V,H]."""
  if h.is_cuda and h.dtype == torch.bfloat16:
    return _LMHeadLoss.apply(h.contiguous(), w, targets, ignore_id, logit_scale, chunk_rows)
  return R.lm_head_loss(h, w, targets.reshape(-1), ignore_id, logit_scale)
