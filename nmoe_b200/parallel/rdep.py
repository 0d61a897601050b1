"""RDEP expert parallelism: routing plan, direct placement into the owner's peer-mapped
buffer, grouped expert GEMMs on the owner, gate-weighted return into the source's
(token, slot) buffer and a fixed-order reduce.  No all-to-all collective; row counts stay on the
device and the grouped GEMMs read them from there.  Host synchronisation: none on one GPU and none with
a capacity factor; with lossless buffers on several GPUs, one 4-byte read per MoE forward sizes the
layer's activations to the rows that actually arrived (see ``Rdep.trim_rows``).

``Rdep.moe(x, gates, eid, W13, W2)`` is the differentiable entry point
(reference: nmoe/rdep.py:34-145 and the autograd functions in nmoe/moe.py:52-617).

Expert weight layout (chosen so that every forward GEMM reads a K-major B operand):
  W13 [n_local, 2*Dff, H]   row 2j = gate projection j, row 2j+1 = up projection j
  W2  [n_local, H, Dff]
``to_reference_layout`` / ``from_reference_layout`` convert to the reference's
W1,W3 [E,H,Dff], W2 [E,Dff,H] (nmoe/model.py:92-94) for checkpoints.
"""
from __future__ import annotations

import collections
import ctypes
import os
import sys
from dataclasses import dataclass
from typing import Optional, Tuple

import torch
import torch.distributed as dist

from ..ops import _lib as L
from ..ops import elementwise as EW
from ..ops import tc_gemm as G
from ..metrics import span
from ..ref import ops as R
from .peer import PeerSlab


def to_reference_layout(W13: torch.Tensor, W2: torch.Tensor):
  W1 = W13[:, 0::2, :].transpose(1, 2).contiguous()
  W3 = W13[:, 1::2, :].transpose(1, 2).contiguous()
  return W1, W3, W2.transpose(1, 2).contiguous()


def from_reference_layout(W1: torch.Tensor, W3: torch.Tensor, W2: torch.Tensor):
  E, H, F = W1.shape
  W13 = torch.empty(E, 2 * F, H, dtype=W1.dtype, device=W1.device)
  W13[:, 0::2, :] = W1.transpose(1, 2)
  W13[:, 1::2, :] = W3.transpose(1, 2)
  return W13, W2.transpose(1, 2).contiguous()


@dataclass
class Plan:
  """Device-resident routing plan of one MoE call (kept for the backward re-dispatch)."""
  eid: torch.Tensor            # [T*K] int32 global expert ids
  rank_in_block: torch.Tensor  # [T*K]
  block_prefix: torch.Tensor   # [n_blocks, E]
  base: torch.Tensor           # [E]
  offs_pad: torch.Tensor       # [n_local+1]
  seg_rows: torch.Tensor       # [n_local]
  tile_expert: torch.Tensor    # [cap/128]
  n_m_tiles: torch.Tensor      # [1]
  send_counts: torch.Tensor    # [E]
  send_prefix: torch.Tensor    # [E] row of this rank's first pair of expert e in its own return buffer
  runs: torch.Tensor           # [3, n_local, world] owner side: run start / length / start at the source (see csrc/rdep.cu)
  pos: torch.Tensor            # [T*K] position in the owner's buffer (-1 = dropped)
  lpos: torch.Tensor           # [T*K] row of the pair in this rank's return buffer (-1 = dropped)
  T: int
  K: int
  rows: int = 0                # host-known bound on the (padded) rows that landed on this rank; 0 = not read back


class Rdep:
  """Shared by all MoE layers of a model: peer slab, scratch, epochs."""

  def __init__(self, dim: int, n_experts: int, topk: int, max_tokens: int, *, capacity_factor: float = 0.0,
               group: Optional[dist.ProcessGroup] = None, device: Optional[torch.device] = None,
               profile: str = "bf16", single_process: bool = False):
    # single_process: every expert lives on this GPU even when a process group exists (each rank of a
    # serving job runs its own replica of the grading model)
    multi = dist.is_initialized() and not single_process
    self.world = dist.get_world_size(group) if multi else 1
    self.rank = dist.get_rank(group) if multi else 0
    assert n_experts % self.world == 0
    self.group = group
    self._capacity_factor, self._profile, self._single_process = capacity_factor, profile, single_process
    self.halves: Optional[list] = None          # see make_halves()
    self.pipe_streams: list = []
    self.pipe_min_tokens = int(os.environ.get("NMOE_MOE_PIPELINE_MIN_TOKENS", "1024"))
    self.dim, self.E, self.K = dim, n_experts, topk
    self.n_local = n_experts // self.world
    self.max_tokens = max_tokens
    self.device = device or torch.device("cuda", torch.cuda.current_device())
    pairs = max_tokens * topk
    worst = pairs * self.world
    avg = pairs
    # capacity_factor <= 0: room for every pair of every rank landing here (lossless, the reference's
    # sizing: nmoe/model.py:203-204); > 0: that multiple of the balanced share, rows beyond it are
    # dropped and reported through the status record
    rows = worst if (self.world == 1 or capacity_factor <= 0) else min(worst, int(avg * capacity_factor))
    # per-expert segments are padded to `align` rows: 256 lets the grouped GEMMs run on CTA pairs (two-SM MMA)
    # "nvfp4x16" (NVFP4 proper): rows travel and are kept in bf16 like the bf16 profile, and are quantised on the owner
    self.nv16 = profile == "nvfp4x16"
    if self.nv16:
      profile = "bf16"
    self.align = 256 if (G.PAIR_MODE and profile == "bf16") else 128
    if os.environ.get("NMOE_RDEP_ALIGN"):
      self.align = int(os.environ["NMOE_RDEP_ALIGN"])
    self.capacity = ((rows + self.n_local * (self.align - 1) + 255) // 256) * 256
    H = dim
    regions = [
      ("x", self.capacity * H * 2), ("y", self.capacity * H * 2), ("meta", self.capacity * 16),
      ("counts", self.world * self.E * 4), ("count_flags", 64), ("data_flags", 64), ("ret_flags", 64),
      ("ret", pairs * H * 2), ("retg", pairs * 4),
    ]
    self.profile = profile
    if profile != "bf16":
      from ..ops.quant import sf_bytes
      regions += [("xq", self.capacity * H), ("sfa", sf_bytes(self.capacity, H))]
    # NMOE_RDEP_GUARD=<bytes>: canary areas after every peer-visible region (see PeerSlab.check_guards)
    self.slab = PeerSlab(regions, group, local_only=single_process,
                         guard_bytes=int(os.environ.get("NMOE_RDEP_GUARD", "0")))
    self.fp4 =profile in ("nvfp4", "mxfp4", "fp4")
    if profile != "bf16":
      # fp4 rows use the first half of the region (H/2 bytes per row)
      self.xq = (self.slab.local("xq", torch.uint8, (self.capacity, H)).view(-1)[:self.capacity * H // 2].view(self.capacity, H // 2)
                 if self.fp4 else self.slab.local("xq", torch.uint8, (self.capacity, H)))
      self.sfa = self.slab.local("sfa", torch.uint8, (sf_bytes(self.capacity, H),))
    self.xbuf = self.slab.local("x", torch.bfloat16, (self.capacity, H))
    self.ybuf = self.slab.local("y", torch.bfloat16, (self.capacity, H))
    self.ret = self.slab.local("ret", torch.bfloat16, (pairs, H))
    self.retg = self.slab.local("retg", torch.float32, (pairs,))
    self.done_counter = torch.zeros(1, dtype=torch.int32, device=self.device)
    self.epoch_count = 0
    self.epoch_data = 0
    self.epoch_ret = 0
    self.wait_budget = 0          # 0 = library default (seconds); tests shrink it
    # fused_return: the down-projection GEMM's epilogue sends its rows to the sources itself (bulk copies of contiguous
    # runs); False: a local GEMM, then a separate push kernel (NMOE_RDEP_FUSED_RETURN=0/1 overrides).  Default by
    # measurement with the run-ordered return, Moonlight shape, GEMM + return: 531 us against ~800 us at 2 GPUs and
    # 624 us against 1145 us at 4 GPUs (the push kernel alone moves its bytes at 647 GB/s there).
    env = os.environ.get("NMOE_RDEP_FUSED_RETURN", "")
    self.fused_return = (env == "1") if env in ("0", "1") else True
    # unfused return: 1 = rows travel as bulk asynchronous copies (global -> shared -> peer), 0 = 16-byte stores
    self.push_impl = int(os.environ.get("NMOE_RDEP_PUSH_BULK", "1"))
    self.fused_swiglu_quant = True  # block-scaled profiles: SwiGLU + quantise in the up/gate GEMM's epilogue
    # world > 1, lossless sizing: the receive buffers hold the worst case (world x the balanced share), but every
    # per-layer tensor derived from them (H13, activations, their gradients) only needs the rows that arrived.
    # Reading that one number back costs one small host read per MoE forward (the shared-expert MLP is already
    # queued on its own stream by then, so the device does not idle) and cuts those tensors by ~world x.
    # With a capacity factor the buffers themselves are a small multiple of the balanced share: nothing is read
    # back and the layer runs without any host synchronisation, at the price of dropping rows beyond that bound.
    self.trim_rows = (self.world > 1 or os.environ.get("NMOE_RDEP_TRIM") == "1") and capacity_factor <= 0
    # start the mark a little above the balanced share (pairs + half a tile of padding per expert), on a 4096-row grid
    # NMOE_RDEP_ROWS: "stale" (default) sizes them from the mark without reading anything back; "exact" reads the
    # count of every call (one 4-byte host read per MoE forward) and can never fall short
    self.rows_mode = os.environ.get("NMOE_RDEP_ROWS", "stale")
    self.rows_overflows = 0
    self.rows_last = 0            # padded expert rows of the newest call whose count has reached the host
    self.rows_dropped = 0         # rows that calls skipped because they did not fit the bound, since the start
    self._seen = torch.full((256,), -1, dtype=torch.int32).pin_memory() if self.device.type == "cuda" else None
    self._seen_next = 0
    self._seen_pending = collections.deque()
    self._rows_grain = 4096
    start = int(1.06 * pairs) + self.n_local * self.align // 2
    self._rows_hwm = min(self.capacity, (start + self._rows_grain - 1) // self._rows_grain * self._rows_grain)
    # world > 1 (bf16): keep a copy of the dispatched rows for the weight gradient instead of sending x over
    # NVLink a second time in backward (one of five transfers per layer; costs rows x H x 2 bytes per layer)
    self.save_dispatched = self.world > 1

  # ---------------------------------------------------------------- building blocks
  def rows_of(self, plan: Plan) -> int:
    """Rows of the expert-side buffers that the layer's tensors must cover (multiple of 256)."""
    if plan.rows == 0:
      if self.trim_rows and self.rows_mode == "stale":
        # no host read: size by the mark, let a one-thread kernel cut the device-side tile count to it and leave the true
        # count in pinned memory, which the host looks at on later calls (see _poll_seen)
        self._poll_seen()
        limit = min(self.capacity, self._rows_hwm)
        slot = self._seen_next
        self._seen_next = (slot + 1) % self._seen.numel()
        self._seen[slot] = -1
        L.check(L.lib().nmoe_rdep_clamp_tiles(L.ptr(plan.n_m_tiles), limit // 128,
                                              ctypes.c_void_p(self._seen.data_ptr() + 4 * slot), L.stream()), "rdep_clamp_tiles")
        self._seen_pending.append((slot, limit // 128))
        plan.rows = limit
      elif self.trim_rows:
        n = int(plan.n_m_tiles.item()) * 128
        # Not the exact count but a high-water mark on a coarse grid: the per-layer tensors then have the SAME size in
        # every layer and step (until routing sets a new maximum), so the caching allocator hands the same blocks round
        # instead of meeting a new size in every layer of every step -- which it answers with cudaMalloc / cudaFree for
        # the first dozens of steps (measured at 4 GPUs: 462 ms per step while that lasts, 394 ms after).
        self._rows_hwm = max(self._rows_hwm, (n + self._rows_grain - 1) // self._rows_grain * self._rows_grain)
        plan.rows = min(self.capacity, self._rows_hwm)
      else:
        plan.rows = self.capacity
    return plan.rows

  def _poll_seen(self) -> None:
    """Look at the row counts that earlier calls left in pinned memory (those whose kernel has run by now): a count
    near the mark raises the mark before it is hit; a count above the limit it was given means that call computed only
    the rows that fitted -- reported once per occurrence, and the mark jumps past it."""
    while self._seen_pending:
      slot, limit_tiles = self._seen_pending[0]
      n = int(self._seen[slot])
      if n < 0:
        break                                   # that kernel has not run yet; later entries have not either
      self._seen_pending.popleft()
      self.rows_last = n * 128
      if n > limit_tiles:
        self.rows_overflows += 1
        self.rows_dropped += (n - limit_tiles) * 128
        print(f"[nmoe] rank {self.rank}: {n * 128} expert rows arrived where {limit_tiles * 128} were provided for; "
              f"{(n - limit_tiles) * 128} rows of that call were not computed (raising the bound)", file=sys.stderr, flush=True)
      need = n * 128
      if need > 0.92 * self._rows_hwm:
        g = self._rows_grain
        self._rows_hwm = min(self.capacity, (int(need * 1.08) + g - 1) // g * g)

  def comm_counters(self) -> dict:
    """Host-side counters of the dispatch path for the metrics store (``comm/*``, nmoe/metrics.py:355-381): rows
    received by this rank in the newest call whose count is known, the receive capacity and its utilisation, the
    current row bound, and rows dropped since the start.  Reads nothing from the device."""
    return {"M_recv": float(self.rows_last), "capacity": float(self.capacity),
            "capacity_utilization": self.rows_last / self.capacity if self.capacity else 0.0,
            "row_bound": float(min(self.capacity, self._rows_hwm)), "dropped_rows": float(self.rows_dropped),
            "overflow_calls": float(self.rows_overflows)}

  def plan(self, eid: torch.Tensor) -> Plan:
    T, K = eid.shape
    assert T <= self.max_tokens and K == self.K
    dev = eid.device
    n_pairs = T * K
    lib = L.lib()
    e32 = eid.reshape(-1).to(torch.int32).contiguous()
    nb = lib.nmoe_rdep_count_blocks(n_pairs)
    block_hist = torch.empty(max(nb, 1), self.E, dtype=torch.int32, device=dev)
    rib = torch.empty(n_pairs, dtype=torch.int32, device=dev)
    st = G.status_buffer(dev)
    L.check(lib.nmoe_rdep_count(L.ptr(e32), n_pairs, self.E, L.ptr(block_hist), L.ptr(rib), L.ptr(st), L.stream()),
            "rdep_count")
    nlw = self.n_local * self.world
    small = torch.empty(self.E * 3 + 2 * self.n_local + 2 + 3 * nlw + self.capacity // 128, dtype=torch.int32, device=dev)
    o = 0
    base = small[o:o + self.E]; o += self.E
    send_counts = small[o:o + self.E]; o += self.E
    send_prefix = small[o:o + self.E]; o += self.E
    runs = small[o:o + 3 * nlw]; o += 3 * nlw
    offs_pad = small[o:o + self.n_local + 1]; o += self.n_local + 1
    seg_rows = small[o:o + self.n_local]; o += self.n_local
    n_m_tiles = small[o:o + 1]; o += 1
    tile_expert = small[o:o + self.capacity // 128]
    self.epoch_count += 1
    L.check(lib.nmoe_rdep_plan(self.rank, self.world, self.E, self.n_local, nb, self.capacity, self.epoch_count, self.align,
                               L.ptr(block_hist), self.slab.ptrs("counts"), self.slab.ptrs("count_flags"),
                               L.ptr(base), L.ptr(offs_pad), L.ptr(seg_rows), L.ptr(tile_expert), L.ptr(n_m_tiles),
                               L.ptr(send_counts), L.ptr(send_prefix), L.ptr(runs), L.ptr(st), L.stream()), "rdep_plan")
    pos = torch.empty(2 * n_pairs, dtype=torch.int32, device=dev)
    return Plan(e32, rib, block_hist, base, offs_pad, seg_rows, tile_expert, n_m_tiles, send_counts, send_prefix,
                runs.view(3, self.n_local, self.world), pos[:n_pairs], pos[n_pairs:], T, K)

  def place(self, x: torch.Tensor, plan: Plan, gates: Optional[torch.Tensor], which: str, with_meta: bool) -> None:
    """Store x's rows into every owner's ``which`` buffer ('x' or 'y') and release the data flags."""
    self.epoch_data += 1
    st = G.status_buffer(x.device)
    L.check(L.lib().nmoe_rdep_place(
      self.rank, self.world, self.E, self.n_local, plan.T, plan.K, self.dim, self.epoch_data, L.ptr(x),
      L.ptr(plan.eid), L.ptr(gates), L.ptr(plan.rank_in_block), L.ptr(plan.block_prefix), L.ptr(plan.base),
      self.slab.ptrs(which), self.slab.ptrs("meta") if with_meta else None, self.slab.ptrs("data_flags"),
      L.ptr(plan.pos), None, L.ptr(plan.offs_pad), L.ptr(plan.seg_rows), L.ptr(self.done_counter), L.ptr(st),
      L.ptr(plan.send_prefix), L.ptr(plan.lpos), L.stream()), "rdep_place")

  def place_mx(self, x: torch.Tensor, plan: Plan, gates: Optional[torch.Tensor]) -> None:
    """Quantise x's rows to MXFP8 (or MXFP4) in the placement kernel and store values + scales into the owners' buffers."""
    self.epoch_data += 1
    st = G.status_buffer(x.device)
    L.check(L.lib().nmoe_rdep_place_mx(
      self.rank, self.world, self.E, self.n_local, plan.T, plan.K, self.dim, self.epoch_data, L.ptr(x),
      L.ptr(plan.eid), L.ptr(gates), L.ptr(plan.rank_in_block), L.ptr(plan.block_prefix), L.ptr(plan.base),
      self.slab.ptrs("xq"), self.slab.ptrs("sfa"), self.slab.ptrs("meta"), self.slab.ptrs("data_flags"),
      L.ptr(plan.pos), L.ptr(plan.offs_pad), L.ptr(plan.seg_rows), L.ptr(self.done_counter), L.ptr(st),
      int(self.fp4), L.ptr(plan.send_prefix), L.ptr(plan.lpos), L.stream()), "rdep_place_mx")

  def wait_data(self) -> None:
    st = G.status_buffer(self.device)
    L.check(L.lib().nmoe_rdep_wait(ctypes.c_void_p(self.slab.local_ptr("data_flags")), self.world,
                                   ctypes.c_uint(self.epoch_data), ctypes.c_uint(self.wait_budget), L.ptr(st), 420,
                                   L.stream()), "rdep_wait(data)")

  def push_and_reduce(self, y: Optional[torch.Tensor], plan: Plan, gates: Optional[torch.Tensor],
                      rowval: Optional[torch.Tensor], out: torch.Tensor, marks: Optional[list] = None) -> None:
    """Owner -> source return of rows in runs (and optional per-row scalars), then the source-side K-way sum with
    the gates applied there (``gates`` fp32 [T*K], or None for a plain sum).
    ``marks``: two CUDA events recorded after the push kernel and after the wait (benchmarks)."""
    lib = L.lib()
    st = G.status_buffer(self.device)
    L.check(lib.nmoe_rdep_push(L.ptr(y), L.ptr(plan.runs), L.ptr(plan.tile_expert), L.ptr(plan.n_m_tiles),
                               self.capacity, self.dim, self.slab.ptrs("ret"), self.slab.ptrs("retg"), L.ptr(rowval),
                               self.world, self.n_local, self.max_tokens * self.K, L.ptr(st), self.push_impl,
                               L.stream()), "rdep_push")
    if marks:
      marks[0].record()
    self.finish_return(plan, out, gates, marks[1] if marks else None)

  def push_args(self, plan: Plan, rowval: Optional[torch.Tensor] = None) -> dict:
    """Arguments that make a grouped GEMM's epilogue store its rows straight into the source ranks'
    return buffers (fused return) instead of a local output."""
    return {"runs": plan.runs, "peer_ret": self.slab.ptrs("ret"), "peer_retg": self.slab.ptrs("retg"),
            "rowval": rowval, "pairs": self.max_tokens * self.K, "world": self.world}

  def finish_return(self, plan: Plan, out: torch.Tensor, gates: Optional[torch.Tensor] = None, mark=None) -> None:
    """After a kernel that sent rows to the sources: publish, wait for every owner, sum the K slots (gate-weighted)."""
    lib = L.lib()
    st = G.status_buffer(self.device)
    self.epoch_ret += 1
    L.check(lib.nmoe_rdep_signal(self.slab.ptrs("ret_flags"), self.rank, self.world, ctypes.c_uint(self.epoch_ret),
                                 L.stream()), "rdep_signal")
    L.check(lib.nmoe_rdep_wait(ctypes.c_void_p(self.slab.local_ptr("ret_flags")), self.world,
                               ctypes.c_uint(self.epoch_ret), ctypes.c_uint(self.wait_budget), L.ptr(st), 421,
                               L.stream()), "rdep_wait(ret)")
    if mark is not None:
      mark.record()
    L.check(lib.nmoe_rdep_reduce(ctypes.c_void_p(self.slab.local_ptr("ret")), L.ptr(plan.lpos), L.ptr(gates), L.ptr(out),
                                 plan.T, plan.K, self.dim, L.stream()), "rdep_reduce")

  def returned_scalars(self, plan: Plan) -> torch.Tensor:
    """The per-pair scalars the owners sent back with the last return, in (token, slot) order (0 for dropped pairs)."""
    n = plan.T * plan.K
    out = torch.empty(n, dtype=torch.float32, device=self.device)
    L.check(L.lib().nmoe_rdep_gather_scalar(ctypes.c_void_p(self.slab.local_ptr("retg")), L.ptr(plan.lpos), L.ptr(out), n,
                                            L.stream()), "rdep_gather_scalar")
    return out.view(plan.T, plan.K)

  def row_gates(self, plan: Plan) -> torch.Tensor:
    out = torch.empty(self.capacity, dtype=torch.float32, device=self.device)
    L.check(L.lib().nmoe_rdep_row_gates(ctypes.c_void_p(self.slab.local_ptr("meta")), L.ptr(plan.n_m_tiles),
                                        self.capacity, L.ptr(out), L.stream()), "rdep_row_gates")
    return out

  # ---------------------------------------------------------------- differentiable MoE
  def moe(self, x: torch.Tensor, gates: torch.Tensor, eid: torch.Tensor, W13: torch.Tensor, W2: torch.Tensor,
          save_h13: bool = False, wq: Optional[tuple] = None) -> torch.Tensor:
    """out[t] = sum_k gates[t,k] * Expert_{eid[t,k]}(x[t]); x [T,H] bf16, gates fp32 [T,K], eid [T,K].

    ``wq`` = (W13q, W13sf, W2q, W2sf) selects the block-scaled FP8 forward (tokens are quantised inside
    the placement kernel, both expert GEMMs run on the MXFP8 tensor-core path); the backward stays
    bf16 with a straight-through estimator, like the reference (nmoe/moe.py:404-415)."""
    if self.halves is not None and x.is_cuda and x.size(0) >= 2 * self.pipe_min_tokens \
        and (x.size(0) + 1) // 2 <= self.halves[0].max_tokens:
      return _MoEPipelined.apply(self, x, gates, eid, W13, W2, save_h13, wq)
    return _MoEFused.apply(self, x, gates, eid, W13, W2, save_h13, wq)

  def make_halves(self) -> None:
    """Collective (every rank of the group must call it at the same point): two more instances, each sized for half of
    ``max_tokens`` with its own peer buffers and flags, and two streams.  ``moe`` then runs the halves of a call
    side by side (``_MoEPipelined``)."""
    if self.halves is not None:
      return
    half = (self.max_tokens + 1) // 2
    mk = lambda: Rdep(self.dim, self.E, self.K, half, capacity_factor=self._capacity_factor, group=self.group,
                      device=self.device, profile=self._profile, single_process=self._single_process)
    self.halves = [mk(), mk()]
    for h in self.halves:
      h.fused_return, h.push_impl, h.wait_budget = self.fused_return, self.push_impl, self.wait_budget
    self.pipe_streams = [torch.cuda.Stream(device=self.device), torch.cuda.Stream(device=self.device)]

  def close(self) -> None:
    for h in (self.halves or []):
      h.close()
    self.slab.close()


def _moe_forward(rdep: "Rdep", x, gates32, eid, W13, W2, save_h13, wq, out):
  """Forward of the routed experts for the tokens of ``x`` on the current stream, result into ``out`` (same shape as
  x).  Returns (plan, h13 kept for backward or None, dispatched rows kept for backward or None)."""
  plan = rdep.plan(eid)
  rows = rdep.rows_of(plan)
  if wq is not None and rdep.nv16:
    # NVFP4 proper: bf16 rows are placed as in the bf16 profile, quantised on the owner (16-element blocks, UE4M3 scales,
    # fixed activation tensor scale), both projections on the kind::mxf4nvf4 scale_vec::4X tensor-core path
    from ..ops import quant as Q
    W13q, W13sf, a13, W2q, W2sf, a2 = wq
    ts = Q.nvfp4_act_scale(x.device)
    with span("time_ms/comm/rdep_dispatch"):
      rdep.place(x, plan, gates32.view(-1), "x", with_meta=True)
      rdep.wait_data()
    xq, xsf = Q.quant_nvfp4_rows(rdep.xbuf[:rows], ts)
    h13 = Q.grouped_gemm_nvfp4(xq, xsf, W13q, W13sf, a13, plan.tile_expert, plan.n_m_tiles)
    a = EW.swiglu_rows(h13, plan.n_m_tiles)
    aq, asf = Q.quant_nvfp4_rows(a, ts)
    y = Q.grouped_gemm_nvfp4(aq, asf, W2q, W2sf, a2, plan.tile_expert, plan.n_m_tiles)
    rdep.push_and_reduce(y, plan, gates32.view(-1), None, out)
    xd = rdep.xbuf[:rows].clone() if rdep.save_dispatched else None
    return plan, (h13 if save_h13 else None), xd
  if wq is not None:
    from ..ops import quant as Q
    W13q, W13sf, W2q, W2sf = wq
    with span("time_ms/comm/rdep_dispatch"):
      rdep.place_mx(x, plan, gates32.view(-1))
      rdep.wait_data()
    ggemm = Q.grouped_gemm_mxfp4 if rdep.fp4 else Q.grouped_gemm_mxfp8
    if not rdep.fused_swiglu_quant:
      h13 = ggemm(rdep.xq[:rows], rdep.sfa, W13q, W13sf, plan.tile_expert, plan.n_m_tiles)
      aq, asf = (Q.swiglu_quant_mxfp4 if rdep.fp4 else Q.swiglu_quant_mxfp8)(h13, plan.n_m_tiles)
    elif save_h13:
      # one epilogue pass writes both the quantised activation and the bf16 H13 that the backward keeps
      aq, asf, h13 = Q.grouped_gemm_swiglu_quant(rdep.xq[:rows], rdep.sfa, W13q, W13sf, plan.tile_expert,
                                                 plan.n_m_tiles, fp4=rdep.fp4, want_h13=True)
    else:
      # SwiGLU and the re-quantisation happen in the epilogue of the up/gate projection: H13 is never written
      h13 = None
      aq, asf = Q.grouped_gemm_swiglu_quant(rdep.xq[:rows], rdep.sfa, W13q, W13sf, plan.tile_expert, plan.n_m_tiles, fp4=rdep.fp4)
    if rdep.fused_return:
      ggemm(aq, asf, W2q, W2sf, plan.tile_expert, plan.n_m_tiles, push=rdep.push_args(plan))
      rdep.finish_return(plan, out, gates32.view(-1))
    else:
      y = ggemm(aq, asf, W2q, W2sf, plan.tile_expert, plan.n_m_tiles)
      rdep.push_and_reduce(y, plan, gates32.view(-1), None, out)
    return plan, (h13 if save_h13 else None), None
  with span("time_ms/comm/rdep_dispatch"):
    rdep.place(x, plan, gates32.view(-1), "x", with_meta=True)
    rdep.wait_data()
  h13 = G.grouped_gemm(rdep.xbuf[:rows], W13, plan.tile_expert, plan.n_m_tiles, align256=rdep.align == 256)
  a = EW.swiglu_rows(h13, plan.n_m_tiles)
  if rdep.fused_return:
    # down projection whose epilogue stores its rows straight into the sources' return buffers
    G.grouped_gemm(a, W2, plan.tile_expert, plan.n_m_tiles, push=rdep.push_args(plan), align256=rdep.align == 256)
    rdep.finish_return(plan, out, gates32.view(-1))
  else:
    y = G.grouped_gemm(a, W2, plan.tile_expert, plan.n_m_tiles, align256=rdep.align == 256)
    rdep.push_and_reduce(y, plan, gates32.view(-1), None, out)
  xd = rdep.xbuf[:rows].clone() if rdep.save_dispatched else None
  return plan, (h13 if save_h13 else None), xd


def _moe_backward(rdep: "Rdep", plan: Plan, x, gates32, W13, W2, h13, xd, dout, dx, dW13=None, dW2=None, *,
                  accumulate: bool = False, before_wgrad=None, after_wgrad=None):
  """Backward of ``_moe_forward`` on the current stream: dx into ``dx``.  The weight gradients go to fresh tensors, or
  into ``dW13`` / ``dW2`` when given (overwritten, or added to with ``accumulate``: the second half of a pipelined
  layer).  ``before_wgrad`` / ``after_wgrad``: events waited for / recorded around the two weight-gradient GEMMs.
  Returns (dgates [T,K], dW13, dW2)."""
  if xd is None:
    rdep.place(x, plan, gates32.view(-1), "x", with_meta=True)
    rdep.place(dout, plan, None, "y", with_meta=False)
  else:
    # the dispatched x rows were kept: only dOut travels, and it carries the row metadata (source, slot, gate)
    rdep.place(dout, plan, gates32.view(-1), "y", with_meta=True)
  rdep.wait_data()
  nt = plan.n_m_tiles
  rows = rdep.rows_of(plan)
  xb, yb = (rdep.xbuf[:rows] if xd is None else xd), rdep.ybuf[:rows]
  if h13 is None:
    h13 = G.grouped_gemm(xb, W13, plan.tile_expert, nt, align256=rdep.align == 256)
  # dA' = dYe @ W2 (un-gated); the gate enters through the row scale of the SwiGLU backward (optionally the epilogue of
  # that GEMM, NMOE_FUSED_SWIGLU_BWD=1; by default the two kernels, which measured faster)
  row_gate = rdep.row_gates(plan)
  fused = G.grouped_gemm_swiglu_bwd(yb, W2, plan.tile_expert, nt, h13, row_gate, align256=rdep.align == 256)
  if fused is not None:
    dh13, rowdot, a_scaled = fused
  else:
    da = G.grouped_gemm(yb, W2, plan.tile_expert, nt, b_mn=True, align256=rdep.align == 256)
    dh13, rowdot, a_scaled = EW.swiglu_bwd_fused(h13, da, row_gate, True, True, nt)
  # every reader of the peer-written buffers runs before the kernel that returns rows to the sources
  if before_wgrad is not None:
    torch.cuda.current_stream(x.device).wait_event(before_wgrad)
  dW2 = G.grouped_wgrad(yb, a_scaled, plan.offs_pad, rdep.n_local, out=dW2, accumulate=accumulate)       # [E, H, Dff]
  dW13 = G.grouped_wgrad(dh13, xb, plan.offs_pad, rdep.n_local, out=dW13, accumulate=accumulate)         # [E, 2Dff, H]
  if after_wgrad is not None:
    after_wgrad.record(torch.cuda.current_stream(x.device))
  if rdep.fused_return:
    G.grouped_gemm(dh13, W13, plan.tile_expert, nt, b_mn=True, push=rdep.push_args(plan, rowdot), align256=rdep.align == 256)
    rdep.finish_return(plan, dx)
  else:
    dxe = G.grouped_gemm(dh13, W13, plan.tile_expert, nt, b_mn=True, align256=rdep.align == 256)
    rdep.push_and_reduce(dxe, plan, None, rowdot, dx)
  return rdep.returned_scalars(plan), dW13, dW2


class _MoEFused(torch.autograd.Function):
  @staticmethod
  def forward(ctx, rdep: Rdep, x, gates, eid, W13, W2, save_h13, wq=None):
    x = x.contiguous()
    gates32 = gates.detach().float().contiguous()
    out = torch.empty_like(x)
    plan, h13, xd = _moe_forward(rdep, x, gates32, eid, W13, W2, save_h13, wq, out)
    ctx.rdep, ctx.plan = rdep, plan
    ctx.save_for_backward(x, gates32, W13, W2, h13, xd)
    return out

  @staticmethod
  def backward(ctx, dout):
    x, gates32, W13, W2, h13, xd = ctx.saved_tensors
    dx = torch.empty_like(x)
    dg, dW13, dW2 = _moe_backward(ctx.rdep, ctx.plan, x, gates32, W13, W2, h13, xd, dout.contiguous(), dx)
    return None, dx, dg, None, dW13, dW2, None, None


class _MoEPipelined(torch.autograd.Function):
  """The same layer with its tokens cut in two halves that run on two streams, each through its own ``Rdep`` (own
  peer buffers, flags and epochs).  The kernels of one half that only move data between GPUs (placement, return, the
  small waits) then run under the other half's GEMMs instead of in front of them: the dispatch of the second half
  overlaps the up/gate projection of the first, the return of the first overlaps the projections of the second, and the
  same in backward.  Nothing waits on another launch except through stream order and the cross-rank flags the halves
  already use.  The second half ADDS its weight gradients to the first half's (ordered by an event), so no extra
  gradient tensor exists.  This is the coarse (two-chunk) form of consuming dispatched rows while others still arrive."""

  @staticmethod
  def forward(ctx, rdep: Rdep, x, gates, eid, W13, W2, save_h13, wq=None):
    x = x.contiguous()
    gates32 = gates.detach().float().contiguous()
    eid = eid.contiguous()
    T = x.size(0)
    cut = min(rdep.halves[0].max_tokens, (T + 1) // 2)
    bounds = ((0, cut), (cut, T))
    out = torch.empty_like(x)
    main = torch.cuda.current_stream(x.device)
    saved, plans = [], []
    for h, (lo, hi) in enumerate(bounds):
      s = rdep.pipe_streams[h]
      s.wait_stream(main)
      with torch.cuda.stream(s):
        plan, h13, xd = _moe_forward(rdep.halves[h], x[lo:hi], gates32[lo:hi], eid[lo:hi], W13, W2, save_h13, wq, out[lo:hi])
      plans.append(plan)
      saved += [h13, xd]
    for t in (x, gates32, eid, out):
      for s in rdep.pipe_streams:
        t.record_stream(s)
    for s in rdep.pipe_streams:
      main.wait_stream(s)
    ctx.rdep, ctx.plans, ctx.bounds = rdep, plans, bounds
    ctx.save_for_backward(x, gates32, W13, W2, *saved)
    return out

  @staticmethod
  def backward(ctx, dout):
    rdep: Rdep = ctx.rdep
    x, gates32, W13, W2, h13_0, xd_0, h13_1, xd_1 = ctx.saved_tensors
    dout = dout.contiguous()
    main = torch.cuda.current_stream(x.device)
    dx = torch.empty_like(x)
    dg = torch.empty(x.size(0), rdep.K, dtype=torch.float32, device=x.device)
    dW13 = torch.empty_like(W13)
    dW2 = torch.empty_like(W2)
    first_done = torch.cuda.Event()
    for h, (lo, hi) in enumerate(ctx.bounds):
      s = rdep.pipe_streams[h]
      s.wait_stream(main)
      with torch.cuda.stream(s):
        half = rdep.halves[h]
        h13, xd = (h13_0, xd_0) if h == 0 else (h13_1, xd_1)
        if h == 0:
          # fresh weight gradients: the kernels write every element of dW13 / dW2 (experts without rows get zeros)
          g, _, _ = _moe_backward(half, ctx.plans[h], x[lo:hi], gates32[lo:hi], W13, W2, h13, xd, dout[lo:hi], dx[lo:hi],
                                       dW13, dW2, accumulate=False, before_wgrad=None, after_wgrad=first_done)
        else:
          g, _, _ = _moe_backward(half, ctx.plans[h], x[lo:hi], gates32[lo:hi], W13, W2, h13, xd, dout[lo:hi], dx[lo:hi],
                                       dW13, dW2, accumulate=True, before_wgrad=first_done, after_wgrad=None)
        dg[lo:hi].copy_(g)
    for t in (dout, dx, dg, dW13, dW2, x, gates32):
      for s in rdep.pipe_streams:
        t.record_stream(s)
    for s in rdep.pipe_streams:
      main.wait_stream(s)
    return None, dx, dg, None, dW13, dW2, None, None


def moe_reference(x, gates, eid, W13, W2):
  """CPU / oracle statement with the same weight layout."""
  W1, W3, W2r = to_reference_layout(W13, W2)
  return R.moe(x, eid, gates, W1, W3, W2r)
