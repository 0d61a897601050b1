"""Optimizer kernels: flat AdamW over bf16 buffers (``csrc/elementwise.cu``)."""
from __future__ import annotations

import torch

from ..ref import ops as R
from . import _lib as L


def adamw_flat_(p: torch.Tensor, g: torch.Tensor, m: torch.Tensor, v: torch.Tensor, *, lr: float, beta1: float,
                beta2: float, eps: float, weight_decay: float, step: int, grad_scale: float = 1.0) -> None:
  """In-place AdamW on flat contiguous buffers (bf16 storage, fp32 math, decay first)."""
  if p.is_cuda and p.dtype == torch.bfloat16:
    assert p.is_contiguous() and g.is_contiguous() and m.is_contiguous() and v.is_contiguous()
    assert g.dtype == torch.bfloat16 and m.dtype == torch.bfloat16 and v.dtype == torch.bfloat16
    L.check(L.lib().nmoe_adamw_flat(L.ptr(p), L.ptr(g), L.ptr(m), L.ptr(v), L.c_ll(p.numel()), L.c_float(lr),
                                    L.c_float(beta1), L.c_float(beta2), L.c_float(eps), L.c_float(weight_decay),
                                    int(step), L.c_float(grad_scale), L.stream()), "adamw_flat")
    return
  R.adamw_step(p, g.float() * grad_scale, m, v, lr=lr, beta1=beta1, beta2=beta2, eps=eps,
               weight_decay=weight_decay, step=step)


def sumsq(x: torch.Tensor, out: torch.Tensor) -> None:
  """out[0] += sum(x^2) (fp32)."""
  if x.is_cuda and x.dtype == torch.bfloat16 and x.is_contiguous():
    L.check(L.lib().nmoe_sumsq_bf16(L.ptr(x), L.c_ll(x.numel()), L.ptr(out), L.stream()), "sumsq")
  else:
    out += x.float().pow(2).sum()
