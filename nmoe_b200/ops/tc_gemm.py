"""bf16 GEMMs on tcgen05 (``csrc/gemm.cu``): dense, grouped over ragged row segments, and
grouped over ragged contraction ranges (expert wgrad), plus the ``linear`` autograd op.

CPU tensors take the plain-PyTorch statement of the same contraction.
"""
from __future__ import annotations

import os
from typing import Optional

import torch

from . import _lib as L

_STATUS: dict[torch.device, torch.Tensor] = {}


def status_buffer(device: torch.device) -> torch.Tensor:
  """Per-device int32[4] status record that kernels write when a bounded wait runs out."""
  buf = _STATUS.get(device)
  if buf is None:
    buf = torch.zeros(4, dtype=torch.int32, device=device)
    _STATUS[device] = buf
  return buf


def check_status(device: Optional[torch.device] = None) -> None:
  """Synchronising check of the status record(s); raises if any kernel reported a failure."""
  for dev, buf in _STATUS.items():
    if device is not None and dev != device:
      continue
    rec = buf.tolist()
    if rec[0] != 0:
      buf.zero_()
      raise L.NativeLibraryError(f"kernel reported status code={rec[0]} where={rec[1]} a={rec[2]} b={rec[3]} on {dev}")


def check_status_collective(device: Optional[torch.device] = None, world: int = 1, group=None) -> None:
  """``check_status`` for a point where every rank must agree before something irreversible happens (a checkpoint
  is finalised, a run starts): raises on EVERY rank when ANY rank's kernels reported a failure, so no rank goes on
  to write its share of a checkpoint that another rank's stale parameters would poison."""
  err = None
  try:
    check_status(device)
  except L.NativeLibraryError as e:
    err = e
  import torch.distributed as dist
  if world > 1 and dist.is_available() and dist.is_initialized():
    on_cuda = device is not None and device.type == "cuda" and dist.get_backend(group) == "nccl"
    flag = torch.tensor([1 if err is not None else 0], dtype=torch.int32, device=device if on_cuda else "cpu")
    dist.all_reduce(flag, op=dist.ReduceOp.MAX, group=group)
    if err is None and int(flag.item()) != 0:
      err = L.NativeLibraryError("a peer rank's kernels reported a failure (bounded wait ran out or rows were dropped)")
  if err is not None:
    raise err


class StatusWatch:
  """Looks at the status record after every step without making the host wait for the device: ``enqueue()`` copies
  the record into pinned host memory behind the step's kernels, ``poll()`` raises for any earlier copy that has
  arrived with a failure code.  A failure is therefore seen one step late at most, and no step pays a sync."""

  def __init__(self, device: torch.device, depth: int = 4):
    self.device = device
    self.cuda = device.type == "cuda"
    self.host = [torch.zeros(4, dtype=torch.int32) for _ in range(depth)]
    if self.cuda:
      self.host = [h.pin_memory() for h in self.host]
    self.events = [None] * depth
    self.i = 0

  def _examine(self, k: int) -> None:
    self.events[k] = None
    rec = self.host[k].tolist()
    if rec[0] != 0:
      status_buffer(self.device).zero_()
      raise L.NativeLibraryError(f"kernel reported status code={rec[0]} where={rec[1]} a={rec[2]} b={rec[3]} on {self.device}")

  def enqueue(self) -> None:
    k = self.i
    self.i = (self.i + 1) % len(self.host)
    if self.events[k] is not None:
      self.events[k].synchronize()
      self._examine(k)
    self.host[k].copy_(status_buffer(self.device), non_blocking=True)
    if self.cuda:
      ev = torch.cuda.Event()
      ev.record()
      self.events[k] = ev
    else:
      self.events[k] = True

  def poll(self) -> None:
    for k, ev in enumerate(self.events):
      if ev is None:
        continue
      if ev is True or ev.query():
        self._examine(k)


PAIR_MODE = os.environ.get("NMOE_GEMM_PAIR", "1") == "1"
PAIR_PUSH = os.environ.get("NMOE_PAIR_PUSH", "1") == "1"      # fused-return grouped GEMMs on CTA pairs too


def use_pair(M: int, N: int) -> bool:
  """The two-SM kernel (256x256 tiles, csrc/gemm2.cu) pays off once there are enough full tiles."""
  return PAIR_MODE and M >= 512 and N >= 256 and N % 8 == 0


def _rows(t: torch.Tensor) -> int:
  return t.numel() // t.size(-1)


def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False,
         out: Optional[torch.Tensor] = None, out_dtype: torch.dtype = torch.bfloat16, accumulate: bool = False,
         bn: int = 0) -> torch.Tensor:
  """C[M,N] = op(A) @ op(B).

  ``a``: [M,K] (a_mn False) or [K,M] (a_mn True).  ``b``: [N,K] (b_mn False, the nn.Linear
  weight layout) or [K,N] (b_mn True).  Both 2-D with a dense last dim.
  """
  if not a.is_cuda:
    A = a.t() if a_mn else a
    Bm = b if b_mn else b.t()
    c = (A.float() @ Bm.float())
    if out is not None:
      out.copy_(out.float() + c if accumulate else c)
      return out
    return c.to(out_dtype)
  assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16
  assert a.dim() == 2 and b.dim() == 2 and a.stride(1) == 1 and b.stride(1) == 1
  M, K = (a.size(1), a.size(0)) if a_mn else (a.size(0), a.size(1))
  N = b.size(1) if b_mn else b.size(0)
  assert (b.size(0) if b_mn else b.size(1)) == K, f"contraction mismatch {a.shape} {b.shape}"
  if out is None:
    assert not accumulate
    out = torch.empty(M, N, dtype=out_dtype, device=a.device)
  assert out.stride(1) == 1 and out.shape == (M, N)
  # TMA wants every row stride a multiple of 16 bytes.  Tiny projections (a per-head scalar gate: 4 outputs) break that
  # in one of their backward products; pad the offending extent with zeros (a copy of a thin operand).
  if K % 8 and not (a_mn and b_mn):
    r = (-K) % 8
    a = torch.nn.functional.pad(a, (0, 0, 0, r) if a_mn else (0, r))
    b = torch.nn.functional.pad(b, (0, 0, 0, r) if b_mn else (0, r))
    K += r
  if a.stride(0) % 8:
    a = torch.nn.functional.pad(a, (0, (-a.size(1)) % 8)) if a.size(1) % 8 else a.contiguous()
  if b.stride(0) % 8:
    b = torch.nn.functional.pad(b, (0, (-b.size(1)) % 8)) if b.size(1) % 8 else b.contiguous()
  st = status_buffer(a.device)
  if bn == 0 and use_pair(M, N):
    L.check(L.lib().nmoe_gemm_bf16_pair(
      L.ptr(a), L.ptr(b), L.ptr(out), M, N, K, L.c_ll(a.stride(0)), L.c_ll(b.stride(0)), L.c_ll(out.stride(0)),
      int(a_mn), int(b_mn), 0, 1, None, None, None, L.c_ll(a.size(0)), L.c_ll(b.size(0)),
      int(out.dtype == torch.float32), int(accumulate), L.ptr(st), L.stream()), "gemm_bf16_pair")
    return out
  L.check(L.lib().nmoe_gemm_bf16(
    L.ptr(a), L.ptr(b), L.ptr(out), M, N, K, L.c_ll(a.stride(0)), L.c_ll(b.stride(0)), L.c_ll(out.stride(0)),
    int(a_mn), int(b_mn), 0, 1, None, None, None, L.c_ll(a.size(0)), L.c_ll(b.size(0)),
    int(out.dtype == torch.float32), int(accumulate), bn, L.ptr(st), None, None, None, None, 0, 0, L.stream()),
    "gemm_bf16")
  return out


def grouped_gemm(a: torch.Tensor, b: torch.Tensor, tile_expert: torch.Tensor, n_m_tiles: torch.Tensor, *,
                 b_mn: bool = False, out: Optional[torch.Tensor] = None, offs: Optional[torch.Tensor] = None,
                 bn: int = 0, push: Optional[dict] = None, align256: bool = False) -> Optional[torch.Tensor]:
  """Rows of ``a`` [Mcap,K] are 128-aligned per-expert segments; row tile i belongs to expert
  ``tile_expert[i]`` and only the first ``n_m_tiles[0]`` tiles are valid.  ``b``: [E,N,K]
  (b_mn False) or [E,K,N] (b_mn True).  Returns [Mcap,N]; rows past the valid tiles are
  left untouched.  ``offs`` ([E+1] row offsets) is only used by the CPU statement.
  """
  E = b.size(0)
  N = b.size(2) if b_mn else b.size(1)
  K = a.size(1)
  if not a.is_cuda:
    c = torch.zeros(a.size(0), N, dtype=a.dtype) if out is None else out
    nt = int(n_m_tiles.item())
    for i in range(nt):
      e = int(tile_expert[i])
      w = b[e] if b_mn else b[e].t()
      c[i * 128:(i + 1) * 128] = (a[i * 128:(i + 1) * 128].float() @ w.float()).to(c.dtype)
    return c
  assert a.is_contiguous() and b.is_contiguous() and a.size(0) % 128 == 0
  st = status_buffer(a.device)
  b2_rows = E * (K if b_mn else N)
  if (push is not None and align256 and bn == 0 and PAIR_MODE and PAIR_PUSH and N >= 256 and N % 64 == 0
      and a.size(0) % 256 == 0):
    # fused RDEP return on CTA pairs (256-row aligned segments)
    L.check(L.lib().nmoe_gemm_bf16_pair_push(
      L.ptr(a), L.ptr(b), None, a.size(0), N, K, L.c_ll(K), L.c_ll(N if b_mn else K), L.c_ll(N),
      0, int(b_mn), 1, E, L.ptr(tile_expert), L.ptr(n_m_tiles), None, L.c_ll(a.size(0)), L.c_ll(b2_rows),
      0, 0, L.ptr(st), L.ptr(push["runs"]), push["peer_ret"], push.get("peer_retg"), L.ptr(push.get("rowval")),
      int(push["pairs"]), push["world"], L.stream()), "grouped_gemm_bf16_pair(push)")
    return None
  if push is not None:
    # fused RDEP return: rows go to the source ranks' return buffers instead of a local C
    L.check(L.lib().nmoe_gemm_bf16(
      L.ptr(a), L.ptr(b), None, a.size(0), N, K, L.c_ll(K), L.c_ll(N if b_mn else K), L.c_ll(N),
      0, int(b_mn), 1, E, L.ptr(tile_expert), L.ptr(n_m_tiles), None, L.c_ll(a.size(0)), L.c_ll(b2_rows),
      0, 0, bn, L.ptr(st), L.ptr(push["runs"]), push["peer_ret"], push.get("peer_retg"), L.ptr(push.get("rowval")),
      int(push["pairs"]), push["world"], L.stream()), "grouped_gemm_bf16(push)")
    return None
  if out is None:
    out = torch.empty(a.size(0), N, dtype=torch.bfloat16, device=a.device)
  if align256 and bn == 0 and PAIR_MODE and N >= 256 and a.size(0) % 256 == 0:
    # segments are 256-row aligned: both CTAs of a pair see one expert, so the two-SM kernel applies
    L.check(L.lib().nmoe_gemm_bf16_pair(
      L.ptr(a), L.ptr(b), L.ptr(out), a.size(0), N, K, L.c_ll(K), L.c_ll(N if b_mn else K), L.c_ll(out.stride(0)),
      0, int(b_mn), 1, E, L.ptr(tile_expert), L.ptr(n_m_tiles), None, L.c_ll(a.size(0)), L.c_ll(b2_rows),
      0, 0, L.ptr(st), L.stream()), "grouped_gemm_bf16_pair")
    return out
  L.check(L.lib().nmoe_gemm_bf16(
    L.ptr(a), L.ptr(b), L.ptr(out), a.size(0), N, K, L.c_ll(K), L.c_ll(N if b_mn else K), L.c_ll(out.stride(0)),
    0, int(b_mn), 1, E, L.ptr(tile_expert), L.ptr(n_m_tiles), None, L.c_ll(a.size(0)), L.c_ll(b2_rows),
    0, 0, bn, L.ptr(st), None, None, None, None, 0, 0, L.stream()), "grouped_gemm_bf16")
  return out


FUSED_SWIGLU_BWD = os.environ.get("NMOE_FUSED_SWIGLU_BWD", "0") == "1"   # off until it measures faster than the two kernels


def grouped_gemm_swiglu_bwd(dy: torch.Tensor, w2: torch.Tensor, tile_expert: torch.Tensor, n_m_tiles: torch.Tensor,
                            h13: torch.Tensor, row_scale: Optional[torch.Tensor], *, want_a: bool = True,
                            align256: bool = False):
  """The expert MLP's dA GEMM with the SwiGLU backward as its epilogue.

  ``dy`` [Mcap, H] (grouped rows), ``w2`` [E, H, F] so that dA = dy @ w2[e] is [Mcap, F]; ``h13`` [Mcap, 2F] (gate in
  even columns).  Returns (dh13 [Mcap, 2F], rowdot [Mcap] fp32 = <swiglu(h13), dA>, a_scaled [Mcap, F] or None), the
  same three tensors as ``grouped_gemm(..., b_mn=True)`` followed by ``ops.swiglu_bwd_fused``; dA itself is never
  written.  Rows past the valid tiles are left untouched.  Returns None when this shape has no fused form
  (the caller then runs the two-kernel form)."""
  E, K, F = w2.size(0), w2.size(1), w2.size(2)
  M = dy.size(0)
  if not (dy.is_cuda and FUSED_SWIGLU_BWD and F % 32 == 0 and h13.size(1) == 2 * F and K % 64 == 0):
    return None
  assert dy.is_contiguous() and w2.is_contiguous() and h13.is_contiguous() and M % 128 == 0 and dy.size(1) == K
  st = status_buffer(dy.device)
  dh = torch.empty_like(h13)
  ao = torch.empty(M, F, dtype=h13.dtype, device=h13.device) if want_a else None
  parts = torch.empty((F + 255) // 256, M, dtype=torch.float32, device=dy.device)
  pair = align256 and PAIR_MODE and F >= 256 and M % 256 == 0
  fn = L.lib().nmoe_gemm_bf16_pair_swiglu_bwd if pair else L.lib().nmoe_gemm_bf16_swiglu_bwd
  L.check(fn(L.ptr(dy), L.ptr(w2), M, F, K, L.c_ll(K), L.c_ll(F), 1, E, L.ptr(tile_expert), L.ptr(n_m_tiles),
             L.c_ll(M), L.c_ll(E * K), L.ptr(h13), L.ptr(dh), L.ptr(ao), L.ptr(row_scale), L.ptr(parts), L.c_ll(M),
             L.ptr(st), L.stream()), "grouped_gemm_swiglu_bwd")
  return dh, parts.sum(0), ao


def grouped_wgrad(a: torch.Tensor, b: torch.Tensor, offs: torch.Tensor, E: int, *,
                  out: Optional[torch.Tensor] = None, accumulate: bool = False, bn: int = 0) -> torch.Tensor:
  """out[e] = a[rows_e]^T @ b[rows_e]  ([E, Ma, Nb]) with rows_e = offs[e]:offs[e+1] (128-aligned).

  Rows of padding inside a segment must be zero in at least one operand.  Experts without
  rows give zeros.
  """
  Ma, Nb = a.size(1), b.size(1)
  if not a.is_cuda:
    c = torch.zeros(E, Ma, Nb, dtype=torch.float32)
    o = offs.tolist()
    for e in range(E):
      c[e] = a[o[e]:o[e + 1]].float().t() @ b[o[e]:o[e + 1]].float()
    if out is not None:
      out.copy_(out.float() + c if accumulate else c)
      return out
    return c.to(a.dtype)
  assert a.is_contiguous() and b.is_contiguous() and a.size(0) == b.size(0)
  if out is None:
    assert not accumulate
    out = torch.empty(E, Ma, Nb, dtype=torch.bfloat16, device=a.device)
  assert out.is_contiguous()
  st = status_buffer(a.device)
  if bn == 0 and use_pair(Ma, Nb):
    L.check(L.lib().nmoe_gemm_bf16_pair(
      L.ptr(a), L.ptr(b), L.ptr(out), Ma, Nb, 0, L.c_ll(Ma), L.c_ll(Nb), L.c_ll(Nb),
      1, 1, 2, E, None, None, L.ptr(offs), L.c_ll(a.size(0)), L.c_ll(b.size(0)),
      int(out.dtype == torch.float32), int(accumulate), L.ptr(st), L.stream()), "grouped_wgrad_bf16_pair")
    return out
  L.check(L.lib().nmoe_gemm_bf16(
    L.ptr(a), L.ptr(b), L.ptr(out), Ma, Nb, 0, L.c_ll(Ma), L.c_ll(Nb), L.c_ll(Nb),
    1, 1, 2, E, None, None, L.ptr(offs), L.c_ll(a.size(0)), L.c_ll(b.size(0)),
    int(out.dtype == torch.float32), int(accumulate), bn, L.ptr(st), None, None, None, None, 0, 0, L.stream()),
    "grouped_wgrad_bf16")
  return out


class _Linear(torch.autograd.Function):
  """y = x @ w^T (+ bias) with w in the [out, in] layout; dgrad and wgrad use the MN-major
  operand forms of the same kernel, so no transpose is ever materialised."""

  @staticmethod
  def forward(ctx, x, w, bias):
    x2 = x.reshape(-1, x.size(-1))
    if not x2.is_contiguous():
      x2 = x2.contiguous()
    y = gemm(x2, w)
    if bias is not None:
      y += bias
    ctx.save_for_backward(x2, w)
    ctx.has_bias = bias is not None
    ctx.xshape = x.shape
    return y.view(*x.shape[:-1], w.size(0))

  @staticmethod
  def backward(ctx, dy):
    x2, w = ctx.saved_tensors
    dy2 = dy.reshape(-1, dy.size(-1))
    if not dy2.is_contiguous():
      dy2 = dy2.contiguous()
    dx = dw = db = None
    if ctx.needs_input_grad[0]:
      dx = gemm(dy2, w, b_mn=True).view(ctx.xshape)            # [M,out] @ [out,in]
    if ctx.needs_input_grad[1]:
      dw = gemm(dy2, x2, a_mn=True, b_mn=True)                 # dy^T [out,M] @ x [M,in]
    if ctx.has_bias and ctx.needs_input_grad[2]:
      db = dy2.float().sum(0).to(dy.dtype)
    return dx, dw, db


def linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
  if x.is_cuda and x.dtype == torch.bfloat16:
    return _Linear.apply(x, w, bias)
  return torch.nn.functional.linear(x, w, bias)
