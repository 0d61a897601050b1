"""Multi-node expert parallelism ("hybrid" mode): what is built here and what is not.

Inside a node every GPU reaches every other one through peer-mapped memory (``parallel/rdep.py``).
Across nodes the reference uses NVSHMEM (IBGDA puts) with one rule that keeps the number of
network endpoints per GPU small: a row for an expert on another node is sent to the GPU with the
SAME local index on that node (the "proxy"), which forwards it to the owner over that node's peer
memory (nmoe/csrc/rdep_nvshmem.cu, per-node proxy routing).

NVSHMEM is not part of this build, so the device path does not exist: ``available()`` is False and
``Rdep`` refuses a world that spans nodes.  What is provided is the host model of the protocol:
``route`` (who carries a row on each hop) and ``simulate_dispatch`` (delivers rows rank by rank
through those hops), which pin the behaviour a future device implementation must reproduce and
are what the CPU tests exercise.  The library exports the entry points such a build would fill in
(``csrc/hybrid_stub.cpp``); they all return "unavailable".
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Sequence, Tuple

from ..ops import _lib as L


def available() -> bool:
  try:
    return bool(L.lib().nmoe_hybrid_available())
  except Exception:
    return False


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
