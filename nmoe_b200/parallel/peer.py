"""Peer-mapped device memory over NVLink: one cudaMalloc'd slab per rank whose CUDA-IPC
handle is exchanged through the process group, so that every rank holds a device
pointer to every peer's slab and kernels can store into (or load from) a peer directly.

world == 1 degenerates to a local slab with itself as its only "peer".
Reference counterpart: nmoe/rdep.py:113-145 + nmoe/csrc/rdep.cu:511-538.
"""
from __future__ import annotations

import ctypes
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from ..ops import _lib as L


class PeerExchangeError(RuntimeError):
  """A rank did not take part in the exchange of peer-memory handles (it exited, or stalled past the group timeout)."""


def exchange_handles(handle: bytes, group: Optional[dist.ProcessGroup] = None) -> List[bytes]:
  """All-gather one opaque handle per rank.  Any failure of the collective -- a peer that exited before the
  exchange, a peer that never arrives within the process-group timeout -- is raised as PeerExchangeError on the
  ranks that did show up, so that start-up ends with a message instead of a hang."""
  world = dist.get_world_size(group)
  gathered: List[Optional[bytes]] = [None] * world
  try:
    dist.all_gather_object(gathered, bytes(handle), group=group)
  except Exception as e:  # gloo / NCCL surface a lost or late peer as RuntimeError / DistBackendError
    raise PeerExchangeError(f"peer handle exchange failed on rank {dist.get_rank(group)}: {type(e).__name__}: "
                            f"{' '.join(str(e).split())[:300]}") from e
  missing = [r for r, h in enumerate(gathered) if not h]
  if missing:
    raise PeerExchangeError(f"peer handle exchange: no handle from ranks {missing}")
  return [bytes(h) for h in gathered]


class PeerSlab:
  """A byte slab carved into named regions at 256-byte-aligned offsets.

  ``ptrs(name)`` returns a ctypes array of ``world`` device pointers (index = rank) to that
  region in every rank's slab; ``local(name, dtype, shape)`` views this rank's region as a tensor.
  """

  GUARD_BYTE = 0xA5

  def __init__(self, regions: List[Tuple[str, int]], group: Optional[dist.ProcessGroup] = None, *,
               local_only: bool = False, guard_bytes: int = 0):
    multi = dist.is_initialized() and not local_only
    self.world = dist.get_world_size(group) if multi else 1
    self.rank = dist.get_rank(group) if multi else 0
    self.offsets: Dict[str, int] = {}
    self.sizes: Dict[str, int] = {}
    # guard_bytes > 0 (debug / tests): a canary area after every region, filled with GUARD_BYTE and checked by
    # check_guards(): a kernel (local or a peer's) that writes past the end of a region shows up by name.
    self.guard_bytes = (max(0, guard_bytes) + 255) & ~255
    off = 0
    for name, nbytes in regions:
      self.offsets[name] = off
      self.sizes[name] = nbytes
      off += ((nbytes + 255) & ~255) + self.guard_bytes
    self.nbytes = max(off, 256)
    lib = L.lib()
    base = ctypes.c_void_p()
    L.check(lib.nmoe_peer_alloc(ctypes.c_size_t(self.nbytes), ctypes.byref(base)), "peer_alloc", 0)
    self.base = base.value
    self.peer_bases: List[int] = [0] * self.world
    self.peer_bases[self.rank] = self.base
    if self.guard_bytes:
      for name in self.offsets:
        self._guard_view(name).fill_(self.GUARD_BYTE)
      torch.cuda.synchronize()
    self._opened: List[int] = []
    if self.world > 1:
      handle = (ctypes.c_ubyte * 64)()
      L.check(lib.nmoe_peer_get_handle(ctypes.c_void_p(self.base), handle), "peer_get_handle", 0)
      gathered = exchange_handles(bytes(handle), group)
      for r, h in enumerate(gathered):
        if r == self.rank:
          continue
        buf = (ctypes.c_ubyte * 64).from_buffer_copy(h)
        p = ctypes.c_void_p()
        L.check(lib.nmoe_peer_open(buf, ctypes.byref(p)), f"peer_open(rank {r})", 0)
        self.peer_bases[r] = p.value
        self._opened.append(p.value)
      dist.barrier(group=group)

  def ptrs(self, name: str, extra_offset: int = 0):
    arr = (ctypes.c_void_p * self.world)()
    for r in range(self.world):
      arr[r] = self.peer_bases[r] + self.offsets[name] + extra_offset
    return arr

  def local_ptr(self, name: str) -> int:
    return self.base + self.offsets[name]

  def local(self, name: str, dtype: torch.dtype, shape: Tuple[int, ...]) -> torch.Tensor:
    """Zero-copy tensor view of this rank's region (kept alive by this object)."""
    n = 1
    for s in shape:
      n *= s
    esz = torch.empty(0, dtype=dtype).element_size()
    assert n * esz <= self.sizes[name], f"region {name} too small"
    return _tensor_from_ptr(self.local_ptr(name), n * esz, self).view(dtype).view(*shape)

  def _guard_view(self, name: str) -> torch.Tensor:
    start = self.local_ptr(name) + self.sizes[name]
    end = self.local_ptr(name) + ((self.sizes[name] + 255) & ~255) + self.guard_bytes
    return _tensor_from_ptr(start, end - start, self)

  def check_guards(self) -> List[str]:
    """Names of this rank's regions whose trailing canary area was overwritten (empty without guards)."""
    if not self.guard_bytes:
      return []
    torch.cuda.synchronize()
    return [name for name in self.offsets if not bool((self._guard_view(name) == self.GUARD_BYTE).all())]

  def close(self) -> None:
    if self.base:
      torch.cuda.synchronize()
      lib = L.lib()
      for p in self._opened:
        lib.nmoe_peer_close(ctypes.c_void_p(p))
      self._opened = []
      lib.nmoe_peer_free(ctypes.c_void_p(self.base))
      self.base = 0


class _CudaArrayView:
  """Minimal ``__cuda_array_interface__`` holder so torch can wrap a raw device pointer."""

  def __init__(self, ptr: int, nbytes: int, owner):
    self.owner = owner
    self.__cuda_array_interface__ = {
      "shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3, "strides": None,
    }


def _tensor_from_ptr(ptr: int, nbytes: int, owner) -> torch.Tensor:
  return torch.as_tensor(_CudaArrayView(ptr, nbytes, owner), device="cuda")
