"""ZeRO-2 for the replicated (non-expert) parameters.

Each parameter group is flattened once into one bf16 parameter buffer and one bf16 gradient
buffer; parameters and their ``.grad`` become views, so there is no per-step packing copy
(the reference packs with a Python double loop, nmoe/zero2.py:233-253).  Rank r owns shard r
of each buffer and keeps AdamW moments only for it.

Three step implementations with identical math (bf16 moments, fp32 arithmetic, decay first):
  world == 1   one flat AdamW kernel per group
  "nccl"       reduce_scatter_tensor(AVG) -> flat AdamW on the shard -> all_gather_into_tensor
               (the library baseline, nmoe/zero2.py:221-279)
  "fused"      one kernel per group that reads the peers' gradient shards over NVLink, applies
               AdamW and stores the new parameters into every peer's buffer (csrc/zero2.cu)
State-dict keys follow the reference: ``shard_{rank}_{group}_{dtype}`` -> {step, exp_avg, exp_avg_sq}.

Overlap with backward (``zero2_overlap`` / NMOE_ZERO2_OVERLAP=1): every parameter group is cut into buckets of
``zero2_bucket_mb`` in reverse registration order (the order in which backward finishes gradients), each bucket a
flat group of its own with its own shard, moments, ready / done flag rows and completion counter.  A
post-accumulate hook per parameter counts a bucket down; when its last gradient has been written the bucket's step
is queued on a side stream behind an event of the compute stream: announce to the peers, ONE block that waits
(bounded) for their announcements, then the fused kernel, whose own wait passes at once.  Only that one block ever
sits on an SM waiting for a peer, so the compute stream's kernels (which peers may in turn be waiting for) are never
kept off the machine.  ``step()`` runs what backward did not reach, joins the side stream and waits for the peers'
done flags.  Ranks must finish buckets in the same order, as with any bucketed data parallelism; a rank that does
not shows up as a bounded-wait status, not as a hang.  With buckets the shard a rank owns is a slice of every
bucket, so a checkpoint belongs to one bucket size (recorded under ``zero2_layout`` and checked on load).
"""
from __future__ import annotations

import ctypes
import os
from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from .. import ops
from ..config import Config
from ..ops import _lib as L
from ..ops import tc_gemm as G
from ..metrics import span
from .peer import PeerSlab

_ALIGN = 256   # elements; keeps every shard 16-byte aligned and vectorisable


class _FlatGroup:
  def __init__(self, gi: int, group: dict, world: int, rank: int, device: torch.device, dtype: torch.dtype,
               slab: Optional[PeerSlab], slab_prefix: str):
    self.gi, self.name = gi, group["name"]
    self.lr, self.wd = float(group["lr"]), float(group["weight_decay"])
    self.params: List[torch.nn.Parameter] = list(group["params"])
    self.dtype = dtype
    n = sum(p.numel() for p in self.params)
    unit = world * _ALIGN
    self.total = ((n + unit - 1) // unit) * unit
    self.shard = self.total // world
    self.rank, self.world = rank, world
    if slab is not None:
      self.flat_param = slab.local(slab_prefix + "p", dtype, (self.total,))
      self.flat_grad = slab.local(slab_prefix + "g", dtype, (self.total,))
    else:
      self.flat_param = torch.zeros(self.total, dtype=dtype, device=device)
      self.flat_grad = torch.zeros(self.total, dtype=dtype, device=device)
    off = 0
    for p in self.params:
      k = p.numel()
      self.flat_param[off:off + k].copy_(p.data.reshape(-1))
      p.data = self.flat_param[off:off + k].view_as(p.data)
      p.grad = self.flat_grad[off:off + k].view_as(p.data)
      off += k
    self.exp_avg = torch.zeros(self.shard, dtype=dtype, device=device)
    self.exp_avg_sq = torch.zeros(self.shard, dtype=dtype, device=device)
    self.step = 0
    self.pending = 0          # overlap: gradients of this step still to come
    self.launched = False     # overlap: this step's update is already queued

  def relink_grads(self) -> None:
    """Re-point ``.grad`` at the flat buffer (someone may have set it to None)."""
    off = 0
    for p in self.params:
      k = p.numel()
      if p.grad is None or p.grad.data_ptr() != self.flat_grad.data_ptr() + off * self.flat_grad.element_size():
        p.grad = self.flat_grad[off:off + k].view_as(p.data)
      off += k


def bucketize(groups: List[dict], bucket_elems: int) -> List[dict]:
  """Cut every group into buckets of at least ``bucket_elems`` elements, walking its parameters from the last
  registered to the first: backward reaches the late layers' parameters first."""
  if bucket_elems <= 0:
    return groups
  out: List[dict] = []
  for g in groups:
    cur, n = [], 0
    for p in reversed(list(g["params"])):
      cur.append(p)
      n += p.numel()
      if n >= bucket_elems:
        out.append({**g, "params": cur})
        cur, n = [], 0
    if cur:
      out.append({**g, "params": cur})
  return out


class Zero2:
  def __init__(self, groups: List[dict], cfg: Config, *, group: Optional[dist.ProcessGroup] = None):
    self.cfg = cfg
    self.pg = group
    self.world = dist.get_world_size(group) if dist.is_initialized() else 1
    self.rank = dist.get_rank(group) if dist.is_initialized() else 0
    self.betas = (cfg.adam_beta1, cfg.adam_beta2)
    self.eps = cfg.adam_eps
    self.gradnorm_sq: Optional[torch.Tensor] = None
    self.groups: List[_FlatGroup] = []
    live = [g for g in groups if g["params"]]
    if not live:
      self.impl = "none"
      return
    p0 = live[0]["params"][0]
    self.device, dtype = p0.device, p0.dtype
    impl = os.environ.get("NMOE_ZERO2_IMPL", cfg.zero2_impl)
    on_gpu = self.device.type == "cuda" and dtype == torch.bfloat16
    if self.world == 1:
      impl = "single"
    elif impl == "auto":
      impl = "fused" if on_gpu else "nccl"
    self.impl = impl
    env = os.environ.get("NMOE_ZERO2_OVERLAP", "")
    want = getattr(cfg, "zero2_overlap", "auto")
    if env in ("0", "1"):
      want = env == "1"
    elif isinstance(want, str):
      want = (self.world > 1) if want.lower() == "auto" else want.lower() in ("1", "true", "yes", "on")
    self.overlap = bool(want) and on_gpu and impl in ("single", "fused")
    self.bucket_elems = 0
    if self.overlap:
      mb = float(os.environ.get("NMOE_ZERO2_BUCKET_MB", getattr(cfg, "zero2_bucket_mb", 64)))
      self.bucket_elems = max(1, int(mb * (1 << 20) / 2))
      live = bucketize(live, self.bucket_elems)
    slab = None
    if impl == "fused":
      unit = self.world * _ALIGN
      regions = []
      for gi, g in enumerate(live):
        n = sum(p.numel() for p in g["params"])
        tot = ((n + unit - 1) // unit) * unit
        regions += [(f"g{gi}p", tot * 2), (f"g{gi}g", tot * 2)]
      # one 64-byte row of flags per flat group (a row has room for 16 ranks): groups may be in flight together
      regions += [("ready", 64 * len(live)), ("done", 64 * len(live))]
      slab = PeerSlab(regions, group)
      self.done_counter = torch.zeros(len(live), dtype=torch.int32, device=self.device)
    self.slab = slab
    for gi, g in enumerate(live):
      self.groups.append(_FlatGroup(gi, g, self.world, self.rank, self.device, dtype, slab, f"g{gi}"))
    self.side: Optional[torch.cuda.Stream] = None
    self._armed = False
    if self.overlap:
      self.side = torch.cuda.Stream(device=self.device)
      self._events = [torch.cuda.Event() for _ in self.groups]
      for g in self.groups:
        for p in g.params:
          p.register_post_accumulate_grad_hook(self._make_hook(g))

  # ------------------------------------------------------------------ overlap with backward
  def _make_hook(self, g: _FlatGroup):
    def hook(_p: torch.Tensor) -> None:
      if not self._armed or g.launched:
        return
      g.pending -= 1
      if g.pending == 0:
        ev = self._events[g.gi]
        ev.record(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(self.side):
          self.side.wait_event(ev)
          self._update(g, handshake_first=True)
        g.launched = True
    return hook

  # ------------------------------------------------------------------ per-step API
  def set_lrs(self, lrs: Dict[str, float]) -> None:
    for g in self.groups:
      g.lr = lrs["router"] if g.name == "router" else lrs["dense"]

  def zero_grad(self) -> None:
    """Clears the gradient buffers; with overlap it also arms the hooks for ONE backward pass (a loop that
    accumulates several backward passes into one step must leave overlap off)."""
    for g in self.groups:
      g.flat_grad.zero_()
      g.relink_grads()
      g.pending, g.launched = len(g.params), False
    self._armed = self.overlap

  @torch.no_grad()
  def _update(self, g: _FlatGroup, handshake_first: bool = False) -> None:
    """Queue one flat group's step on the current stream (everything but the final wait for the peers)."""
    g.step += 1
    kw = dict(lr=g.lr, beta1=self.betas[0], beta2=self.betas[1], eps=self.eps, weight_decay=g.wd, step=g.step)
    if self.impl == "single":
      if self.gradnorm_sq is not None:
        ops.sumsq(g.flat_grad, self.gradnorm_sq)
      ops.adamw_flat_(g.flat_param, g.flat_grad, g.exp_avg, g.exp_avg_sq, **kw)
    elif self.impl == "nccl":
      lo = self.rank * g.shard
      gshard = torch.empty(g.shard, dtype=g.flat_grad.dtype, device=self.device)
      if g.flat_grad.is_cuda:
        with span("time_ms/zero2_reduce_scatter"):
          dist.reduce_scatter_tensor(gshard, g.flat_grad, op=dist.ReduceOp.AVG, group=self.pg)
      else:  # gloo has no reduce_scatter: all_reduce then slice (CPU tests only)
        full = g.flat_grad.float()
        dist.all_reduce(full, group=self.pg)
        gshard = (full[lo:lo + g.shard] / self.world).to(g.flat_grad.dtype)
      if self.gradnorm_sq is not None:
        ops.sumsq(gshard, self.gradnorm_sq)
      pshard = g.flat_param[lo:lo + g.shard]
      ops.adamw_flat_(pshard, gshard, g.exp_avg, g.exp_avg_sq, **kw)
      if g.flat_param.is_cuda:
        with span("time_ms/zero2_all_gather"):
          dist.all_gather_into_tensor(g.flat_param, pshard.clone(), group=self.pg)
      else:
        parts = [torch.empty_like(pshard) for _ in range(self.world)]
        dist.all_gather(parts, pshard.clone(), group=self.pg)
        g.flat_param.copy_(torch.cat(parts))
    elif self.impl == "fused":
      st = G.status_buffer(self.device)
      lib = L.lib()
      row = 64 * g.gi                                   # this group's row of ready / done flags
      epoch = ctypes.c_uint(g.step)                     # a group's flags count its own steps
      if handshake_first:
        # side stream: announce, then let one block do the waiting, so that the wide kernel below never sits on the
        # SMs waiting for a peer whose own progress may depend on this GPU's compute stream
        L.check(lib.nmoe_rdep_signal(self.slab.ptrs("ready", row), self.rank, self.world, epoch, L.stream()), "zero2_signal")
        L.check(lib.nmoe_rdep_wait(ctypes.c_void_p(self.slab.local_ptr("ready") + row), self.world, epoch,
                                   ctypes.c_uint(0), L.ptr(st), 502, L.stream()), "zero2_ready_wait")
      L.check(lib.nmoe_zero2_fused(
        self.rank, self.world, L.c_ll(g.shard), self.slab.ptrs(f"g{g.gi}g"), self.slab.ptrs(f"g{g.gi}p"),
        self.slab.ptrs("ready", row), self.slab.ptrs("done", row), L.ptr(g.exp_avg), L.ptr(g.exp_avg_sq),
        L.c_float(g.lr), L.c_float(self.betas[0]), L.c_float(self.betas[1]), L.c_float(self.eps),
        L.c_float(g.wd), g.step, L.c_float(1.0 / self.world), epoch, ctypes.c_uint(0),
        ctypes.c_void_p(self.done_counter.data_ptr() + 4 * g.gi), L.ptr(self.gradnorm_sq), L.ptr(st), L.stream()),
        "zero2_fused")
    else:
      raise ValueError(f"unknown zero2 implementation {self.impl!r}")

  @torch.no_grad()
  def step(self) -> None:
    self._armed = False
    fused = self.impl == "fused"
    _t = span("time_ms/zero2_fused") if fused else None    # what backward did not hide: leftovers + the done waits
    if _t is not None:
      _t.__enter__()
    for g in self.groups:
      if not g.launched:
        self._update(g)
      g.launched = False
    if self.side is not None:
      torch.cuda.current_stream(self.device).wait_stream(self.side)
    if fused:
      st = G.status_buffer(self.device)
      for g in self.groups:
        L.check(L.lib().nmoe_rdep_wait(ctypes.c_void_p(self.slab.local_ptr("done") + 64 * g.gi), self.world,
                                       ctypes.c_uint(g.step), ctypes.c_uint(0), L.ptr(st), 501, L.stream()),
                "zero2_wait")
      _t.__exit__(None, None, None)

  # ------------------------------------------------------------------ checkpoint state
  def state_dict(self) -> dict:
    out = {}
    for g in self.groups:
      key = f"shard_{self.rank}_{g.gi}_{str(g.dtype).replace('torch.', '')}"
      out[key] = {"step": g.step, "exp_avg": g.exp_avg, "exp_avg_sq": g.exp_avg_sq}
    out["zero2_layout"] = {"bucket_elems": self.bucket_elems, "totals": [g.total for g in self.groups]}
    return out

  def load_state_dict(self, sd: dict) -> None:
    lay = sd.get("zero2_layout")
    mine = {"bucket_elems": self.bucket_elems, "totals": [g.total for g in self.groups]}
    if lay is not None and (int(lay.get("bucket_elems", 0)) != mine["bucket_elems"] or list(lay.get("totals", [])) != mine["totals"]):
      raise ValueError(f"ZeRO-2 state was written with flat-buffer layout {lay}, this run has {mine}: "
                       "resume with the same zero2_overlap / zero2_bucket_mb")
    for g in self.groups:
      key = f"shard_{self.rank}_{g.gi}_{str(g.dtype).replace('torch.', '')}"
      if key not in sd:
        raise KeyError(f"ZeRO-2 state has no entry {key} (was the checkpoint written with another world size?)")
      g.step = int(sd[key]["step"])
      g.exp_avg.copy_(sd[key]["exp_avg"])
      g.exp_avg_sq.copy_(sd[key]["exp_avg_sq"])
