"""Muon: momentum followed by a Newton-Schulz orthogonalisation of each 2-D update
(reference: the orthogonaliser in nmoe/csrc/muon.cu:288-499, 5 steps of X <- aX + (bA + cA^2)X with
A = X X^T after Frobenius normalisation).  The three matrix products of every step run on the
tcgen05 bf16 GEMM (``ops.gemm``); the quintic coefficients are the usual (3.4445, -4.7750, 2.0315).
"""
from __future__ import annotations

from typing import Dict, List, Tuple

import torch

from ..ref import ops as R
from .tc_gemm import gemm

COEFFS = (3.4445, -4.7750, 2.0315)


@torch.no_grad()
def newton_schulz(x: torch.Tensor, steps: int = 5, coeffs: Tuple[float, float, float] = COEFFS, eps: float = 1e-7) -> torch.Tensor:
  """Approximate orthogonal factor of each matrix in x ([..., M, N]); returns the dtype of x."""
  if not x.is_cuda:
    return R.newton_schulz(x, steps, coeffs, eps)
  a, b, c = coeffs
  shp = x.shape
  X = x.reshape(-1, shp[-2], shp[-1])
  out = torch.empty_like(X, dtype=torch.bfloat16)
  for i in range(X.size(0)):
    m = X[i].float()
    transposed = m.size(0) > m.size(1)
    if transposed:
      m = m.t()
    m = (m / (m.norm() + eps)).bfloat16().contiguous()
    for _ in range(steps):
      A = gemm(m, m)                                   # X X^T                [M, M]
      B = (b * A.float() + c * gemm(A, A).float()).bfloat16()   # A symmetric: A A^T = A^2
      m = (a * m.float() + gemm(B, m, b_mn=True).float()).bfloat16()
    out[i] = m.t() if transposed else m
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
