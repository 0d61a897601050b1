"""Chunked gated delta rule (Kimi Delta Attention) with the sequential part on a CUDA kernel.

Per head, with L2-normalised q and k, per-channel log-decay g_t <= 0 and write strength beta_t:
    S <- diag(exp(g_t)) S ;  S <- S + beta_t k_t (v_t - S^T k_t)^T ;  o_t = S^T (q_t * scale)

Chunk form (C = 64 tokens, everything batched over batch, head and chunk except the state recurrence):
    kd = k * exp(gc), ki = k * exp(-gc), qd = q * exp(gc)          gc = cumulative log-decay inside the chunk
    M  = I + diag(beta) * strict_lower(kd ki^T)
    [U | P] = M^-1 [diag(beta) v | diag(beta) kd]                  one triangular solve for all chunks
    scan:   W_c = U_c - P_c S_c ;  S_{c+1} = diag(exp(g_end)) S_c + (ki * exp(g_end))^T W_c        <- csrc/kda.cu
    o = qd S_c + lower(qd ki^T) W_c

``KdaScan`` is the scan as an autograd function: its backward is the same kernel walked in reverse on transformed
operands (see ``backward``), plus batched products.  CPU tensors (and shapes the kernel does not take) run the same
formulas with a Python loop over chunks, which is also the oracle for the tests.
Reference: nmoe/triton/kda.py:202-1080 (chunked forward / backward, WY representation, state passing).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn.functional as F

from . import _lib as L

CHUNK = 64


def _scan_loop(U, P, K2, dec, G: Optional[torch.Tensor], reverse: bool) -> Tuple[torch.Tensor, torch.Tensor]:
  """Reference statement of the scan: U [BH,n,C,Dv], P/K2 [BH,n,C,Dk], dec [BH,n,Dk], G [BH,n,Dk,Dv] or None
  -> (W [BH,n,C,Dv], S_hist [BH,n,Dk,Dv] = state every chunk was entered with)."""
  BH, n, C, Dv = U.shape
  Dk = P.size(-1)
  S = U.new_zeros(BH, Dk, Dv)
  W = torch.empty_like(U)
  H = U.new_empty(BH, n, Dk, Dv)
  order = range(n - 1, -1, -1) if reverse else range(n)
  for c in order:
    H[:, c] = S
    W[:, c] = U[:, c] - P[:, c] @ S
    S = dec[:, c].unsqueeze(-1) * S + K2[:, c].transpose(1, 2) @ W[:, c]
    if G is not None:
      S = S + G[:, c]
  return W, H


def _kernel_ok(U: torch.Tensor, P: torch.Tensor) -> bool:
  return U.is_cuda and U.dtype == torch.float32 and U.size(2) == CHUNK and U.size(3) % 64 == 0 \
      and P.size(3) % 4 == 0 and P.size(3) <= 256


def scan(U, P, K2, dec, G: Optional[torch.Tensor] = None, reverse: bool = False):
  """The recurrence over chunks (no autograd)."""
  if not _kernel_ok(U, P):
    return _scan_loop(U, P, K2, dec, G, reverse)
  U, P, K2, dec = U.contiguous(), P.contiguous(), K2.contiguous(), dec.contiguous()
  G = G.contiguous() if G is not None else None
  BH, n, C, Dv = U.shape
  Dk = P.size(-1)
  W = torch.empty_like(U)
  H = torch.empty(BH, n, Dk, Dv, dtype=torch.float32, device=U.device)
  L.check(L.lib().nmoe_kda_scan(L.ptr(U), L.ptr(P), L.ptr(K2), L.ptr(dec), L.ptr(G), None, L.ptr(W), L.ptr(H), None,
                                BH, n, Dk, Dv, int(reverse), L.stream()), "kda_scan")
  return W, H


class KdaScan(torch.autograd.Function):
  """(W, S_hist) = scan(U, P, K2, dec), differentiable.

  With lambda_c the gradient of the state chunk c was entered with and omega_c the gradient of W_c:
      omega_c  = dW_c + K2_c lambda_{c+1}
      lambda_c = dS_hist_c + dec_c * lambda_{c+1} - P_c^T omega_c
  which is the same recurrence walked in reverse with U' = dW, P' = -K2, K2' = -P, G = dS_hist; then
      dU = omega,  dP = -omega S^T,  dK2 = W lambda_next^T,  ddec = sum_v lambda_next * S."""

  @staticmethod
  def forward(ctx, U, P, K2, dec):
    W, H = scan(U, P, K2, dec)
    ctx.save_for_backward(P, K2, dec, W, H)
    return W, H

  @staticmethod
  def backward(ctx, dW, dH):
    P, K2, dec, W, H = ctx.saved_tensors
    dW = dW.contiguous() if dW is not None else torch.zeros_like(W)
    dH = dH.contiguous() if dH is not None else torch.zeros_like(H)
    omega, lam_next = scan(dW, -K2, -P, dec, dH, reverse=True)
    dU = omega
    dP = -(omega @ H.transpose(-1, -2))
    dK2 = W @ lam_next.transpose(-1, -2)
    ddec = (lam_next * H).sum(-1)
    return dU, dP, dK2, ddec


def _l2norm(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
  return x * torch.rsqrt(x.pow(2).sum(-1, keepdim=True) + eps)


def kda_chunk_scan(q, k, v, g, beta, scale: Optional[float] = None) -> torch.Tensor:
  """q,k,g [B,T,H,Dk]; v [B,T,H,Dv]; beta [B,T,H] -> o [B,T,H,Dv] fp32.  Differentiable in all five inputs."""
  B, T, H, Dk = q.shape
  Dv = v.size(-1)
  C = CHUNK
  scale = Dk ** -0.5 if scale is None else scale
  pad = (-T) % C
  if pad:
    q, k, v, g = (F.pad(x, (0, 0, 0, 0, 0, pad)) for x in (q, k, v, g))
    beta = F.pad(beta, (0, 0, 0, pad))
  n = (T + pad) // C
  f = lambda x: x.float().reshape(B, n, C, H, -1).permute(0, 3, 1, 2, 4).reshape(B * H, n, C, -1)    # [BH,n,C,D]
  q, k, v, g = f(_l2norm(q.float()) * scale), f(_l2norm(k.float())), f(v), f(g)
  beta = beta.float().reshape(B, n, C, H).permute(0, 3, 1, 2).reshape(B * H, n, C, 1)
  gc = g.cumsum(2)
  kd, ki, qd = k * torch.exp(gc), k * torch.exp(-gc), q * torch.exp(gc)
  strict = torch.tril(torch.ones(C, C, device=q.device), -1)
  incl = torch.tril(torch.ones(C, C, device=q.device))
  M = torch.eye(C, device=q.device) + beta * ((kd @ ki.transpose(-1, -2)) * strict)
  UP = torch.linalg.solve_triangular(M, beta * torch.cat((v, kd), -1), upper=False)
  U, P = UP[..., :Dv], UP[..., Dv:]
  g_end = gc[:, :, -1]                                      # [BH,n,Dk]
  dec = torch.exp(g_end)
  K2 = ki * dec.unsqueeze(2)
  W, S_in = KdaScan.apply(U.contiguous(), P.contiguous(), K2.contiguous(), dec.contiguous())
  o = qd @ S_in + ((qd @ ki.transpose(-1, -2)) * incl) @ W
  o = o.reshape(B, H, n * C, Dv).permute(0, 2, 1, 3)
  return o[:, :T]
