"""Muon: momentum followed by a Newton-Schulz orthogonalisation of each 2-D update
(reference: the orthogonaliser in nmoe/csrc/muon.cu:288-499, 5 steps of X <- aX + (bA + cA^2)X with
A = X X^T after Frobenius normalisation).  The iteration is native (``csrc/muon.cu``): its products run on the
tcgen05 bf16 GEMM (``ops.gemm``); the quintic coefficients are the usual (3.4445, -4.7750, 2.0315).
"""
from __future__ import annotations

import ctypes
from typing import Dict, List, Tuple

import torch

from ..ref import ops as R
from . import _lib as L
from .tc_gemm import status_buffer

COEFFS = (3.4445, -4.7750, 2.0315)


@torch.no_grad()
def newton_schulz(x: torch.Tensor, steps: int = 5, coeffs: Tuple[float, float, float] = COEFFS, eps: float = 1e-7) -> torch.Tensor:
  """Approximate orthogonal factor of each matrix in x ([..., M, N]); returns the dtype of x."""
  if not x.is_cuda:
    return R.newton_schulz(x, steps, coeffs, eps)
  a, b, c = coeffs
  shp = x.shape
  X = x.reshape(-1, shp[-2], shp[-1]).to(torch.bfloat16).contiguous()
  E, Rr, Cc = X.shape
  if Rr % 8 or Cc % 8:
    return R.newton_schulz(x.float(), steps, coeffs, eps).to(x.dtype)
  # the whole iteration runs inside the library (csrc/muon.cu): normalise, then per step three
  # tcgen05 GEMMs with the "a X +" term folded into the last one's accumulate mode
  lib = L.lib()
  lib.nmoe_muon_workspace_elems.restype = ctypes.c_longlong
  ws = torch.empty(lib.nmoe_muon_workspace_elems(Rr, Cc), dtype=torch.bfloat16, device=x.device)
  ssq = torch.empty(E, dtype=torch.float32, device=x.device)
  out = torch.empty_like(X)
  L.check(lib.nmoe_muon_orth(L.ptr(X), L.ptr(out), E, Rr, Cc, int(steps), L.c_float(a), L.c_float(b), L.c_float(c),
                             L.c_float(eps), L.ptr(ws), L.ptr(ssq), L.ptr(status_buffer(x.device)), L.stream()),
          "muon_orth", E * (3 + 5 * steps))
  return out.view(shp).to(x.dtype)


class Muon:
  """Muon for stacks of expert matrices ([E, rows, cols] parameters): Nesterov momentum, Newton-Schulz,
  update scaled by sqrt(max(1, rows/cols)); decoupled weight decay."""

  def __init__(self, params: List[torch.nn.Parameter], lr: float, momentum: float = 0.95, weight_decay: float = 0.0,
               ns_steps: int = 5):
    self.params, self.lr, self.mu, self.wd, self.ns_steps = params, lr, momentum, weight_decay, ns_steps
    self.buf: Dict[int, torch.Tensor] = {i: torch.zeros_like(p) for i, p in enumerate(params)}
    self.step_count = 0

  @torch.no_grad()
  def step(self) -> None:
    for i, p in enumerate(self.params):
      if p.grad is None:
        continue
      g = p.grad
      buf = self.buf[i]
      buf.mul_(self.mu).add_(g)
      u = newton_schulz(g.add(buf, alpha=self.mu), self.ns_steps)
      scale = max(1.0, p.size(-2) / p.size(-1)) ** 0.5
      p.mul_(1.0 - self.lr * self.wd).add_(u.to(p.dtype), alpha=-self.lr * scale)
      p.grad = None
    self.step_count += 1

  def state_dict(self) -> dict:
    return {"step": self.step_count, "state": {i: {"momentum_buffer": b} for i, b in self.buf.items()}}

  def load_state_dict(self, sd: dict) -> None:
    self.step_count = int(sd["step"])
    for i, s in sd["state"].items():
      self.buf[int(i)].copy_(s["momentum_buffer"])
