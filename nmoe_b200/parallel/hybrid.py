"""Multi-node expert parallelism ("hybrid" mode): NVSHMEM across nodes, peer memory inside a node.

Inside a node every GPU reaches every other one through peer-mapped memory (``parallel/rdep.py``).  Across nodes a
row for an expert on another node is put (NVSHMEM, IBGDA where the fabric has it) into the staging buffer of the GPU
with the SAME local index on that node (the "proxy"), which forwards it to the owner over that node's peer memory
(reference: nmoe/csrc/rdep_nvshmem.cu, per-node proxy routing).  One proxy per (sender, node) keeps the number of
network endpoints per GPU at nodes - 1.

Pieces:

* ``csrc/hybrid/rdep_nvshmem.cu`` -> ``lib/libnmoe_hybrid.so`` (built by ``_build.build_hybrid()`` wherever an NVSHMEM
  installation is found: relocatable device code + libnvshmem_device.a): unique-id bootstrap, symmetric allocation,
  ``nmoe_hybrid_dispatch`` (warp-wide non-blocking puts of rows and their records into the sender's own slice of the
  proxy's staging area, fence, one signal per proxy), ``nmoe_hybrid_wait`` (bounded wait on the signals; a status
  record instead of a hang), ``nmoe_hybrid_return`` (outputs straight into the origin's return buffer).
* ``HybridTransport`` below: the Python face of that library (bootstrap through the process group, buffers, calls).
* ``route`` / ``simulate_dispatch``: the host model of the routing rule, which the CPU tests pin.

``Rdep`` itself still refuses a world that spans nodes: wiring the proxy's staged rows into the intra-node placement
is the remaining step, and it cannot be exercised on a single node.  The main library keeps stub entry points
(``csrc/hybrid/hybrid_stub.cpp``) that report "unavailable" when the NVSHMEM library is not loaded.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from pathlib import Path
from typing import Dict, List, Optional, Sequence, Tuple

from ..ops import _lib as L

_HLIB: Optional[ctypes.CDLL] = None


def hybrid_lib() -> Optional[ctypes.CDLL]:
  """The NVSHMEM transport library if it has been built (and its NVSHMEM host library can be loaded), else None."""
  global _HLIB
  if _HLIB is None:
    path = Path(__file__).resolve().parent.parent / "lib" / "libnmoe_hybrid.so"
    if path.exists():
      try:
        _HLIB = ctypes.CDLL(str(path), mode=ctypes.RTLD_GLOBAL)
      except OSError:
        _HLIB = None
  return _HLIB


def available() -> bool:
  lib = hybrid_lib()
  try:
    return bool(lib.nmoe_hybrid_available()) if lib is not None else bool(L.lib().nmoe_hybrid_available())
  except Exception:
    return False


class HybridTransport:
  """Bootstrap and buffers of the inter-node leg.  ``group`` must be a CPU-capable process group spanning all ranks
  (the unique id is broadcast through it).  Buffers are symmetric: the same call with the same size on every rank."""

  def __init__(self, rank: int, world: int, local_world: int, group=None):
    import torch
    import torch.distributed as dist
    lib = hybrid_lib()
    if lib is None:
      raise RuntimeError("the NVSHMEM transport library is not built (python -m nmoe_b200._build --hybrid)")
    if world % local_world:
      raise ValueError("world must be a multiple of local_world")
    self.lib, self.rank, self.world, self.local_world = lib, rank, world, local_world
    n = int(lib.nmoe_hybrid_uid_bytes())
    uid = (ctypes.c_ubyte * n)()
    if rank == 0:
      L.check(lib.nmoe_hybrid_get_uid(uid, ctypes.c_size_t(n)), "hybrid_get_uid", 0)
    box = [bytes(uid)]
    dist.broadcast_object_list(box, src=0, group=group)
    buf = (ctypes.c_ubyte * n).from_buffer_copy(box[0])
    L.check(lib.nmoe_hybrid_init(buf, rank, world, local_world), "hybrid_init", 0)
    self.epoch = 0
    self._bufs: List[int] = []
    self._torch = torch

  def alloc(self, nbytes: int) -> int:
    p = ctypes.c_void_p()
    L.check(self.lib.nmoe_hybrid_alloc(ctypes.c_size_t(nbytes), ctypes.byref(p)), "hybrid_alloc", 0)
    self._bufs.append(p.value)
    return p.value

  def dispatch(self, rows, recs, dst_node, slot, counts, slice_rows: int, staging: int, records: int, signals: int) -> None:
    """rows [n, H] bf16, recs [n, 4] int32 records, dst_node / slot [n] int32, counts [nodes] int32 (device)."""
    self.epoch += 1
    L.check(self.lib.nmoe_hybrid_dispatch(L.ptr(rows), L.ptr(recs), L.ptr(dst_node), L.ptr(slot), L.ptr(counts),
                                          rows.size(0), rows.size(1), slice_rows, self.rank, self.world, self.local_world,
                                          ctypes.c_ulonglong(self.epoch), ctypes.c_void_p(staging),
                                          ctypes.c_void_p(records), ctypes.c_void_p(signals), L.stream()), "hybrid_dispatch")

  def wait(self, signals: int, counts_out, status, budget: int = 0) -> None:
    L.check(self.lib.nmoe_hybrid_wait(ctypes.c_void_p(signals), self.rank, self.world, self.local_world,
                                      ctypes.c_ulonglong(self.epoch), ctypes.c_uint(budget), L.ptr(counts_out),
                                      L.ptr(status), L.stream()), "hybrid_wait")

  def return_rows(self, y, recs, n_pairs: int, ret: int, status) -> None:
    L.check(self.lib.nmoe_hybrid_return(L.ptr(y), L.ptr(recs), y.size(0), y.size(1), self.rank, self.local_world,
                                        n_pairs, ctypes.c_void_p(ret), L.ptr(status), L.stream()), "hybrid_return")

  def quiet(self) -> None:
    L.check(self.lib.nmoe_hybrid_quiet(L.stream()), "hybrid_quiet", 0)

  def barrier(self) -> None:
    L.check(self.lib.nmoe_hybrid_barrier(L.stream()), "hybrid_barrier", 0)

  def close(self) -> None:
    for p in self._bufs:
      self.lib.nmoe_hybrid_free(ctypes.c_void_p(p))
    self._bufs = []
    self.lib.nmoe_hybrid_finalize()


@dataclass(frozen=True)
class Hop:
  src: int
  dst: int
  transport: str      # "local" (same GPU), "peer" (NVLink peer store inside a node), "net" (inter-node put)


def route(src: int, owner: int, local_world: int) -> List[Hop]:
  """Hops a row takes from rank ``src`` to the rank ``owner`` that holds its expert."""
  if src == owner:
    return [Hop(src, owner, "local")]
  if src // local_world == owner // local_world:
    return [Hop(src, owner, "peer")]
  proxy = (owner // local_world) * local_world + src % local_world
  hops = [Hop(src, proxy, "net")]
  if proxy != owner:
    hops.append(Hop(proxy, owner, "peer"))
  return hops


def simulate_dispatch(eid: Sequence[Sequence[int]], n_experts: int, world: int, local_world: int) -> Tuple[Dict[int, List[Tuple[int, int, int]]], Dict[str, int]]:
  """``eid[r]`` = expert ids chosen by rank r's (token, slot) pairs, flattened.  Returns the rows every
  owner ends up with as (source rank, pair index, expert) in arrival-independent (sorted) order, and
  the number of rows carried per transport."""
  n_local = n_experts // world
  inbox: Dict[int, List[Tuple[int, int, int]]] = {r: [] for r in range(world)}
  carried = {"local": 0, "peer": 0, "net": 0}
  for src in range(world):
    for i, e in enumerate(eid[src]):
      owner = e // n_local
      for hop in route(src, owner, local_world):
        carried[hop.transport] += 1
      inbox[owner].append((src, i, e))
  for r in inbox:
    inbox[r].sort(key=lambda t: (t[2], t[0], t[1]))       # expert-major, then source rank, then pair: the plan's order
  return inbox, carried
