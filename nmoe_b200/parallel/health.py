"""Host-side liveness of the ranks of a job, through the rendezvous store.

The expert and ZeRO-2 kernels of one rank wait (bounded) on flags that its peers' kernels write.  When a peer has
died, those waits would each run out and report -- but only after burning their time limit, once per layer.  This
module lets the survivors learn of the loss on the host, BEFORE they launch the next step:

* every rank calls ``beat(step)`` once per step (one small store write),
* a rank that leaves through an exception calls ``fail(reason)`` (``train()`` does this in its handler),
* every rank calls ``check()`` before it launches a step: a peer that has announced its death raises ``PeerLost`` at
  once, a peer whose last beat is older than ``stall_s`` raises ``PeerStalled``.

The store is the process group's own (TCPStore under torchrun, FileStore / HashStore in tests), so no extra ports or
threads are needed.  The reference has no counterpart: its cross-GPU barriers trap the GPU after a cycle budget
(nmoe/csrc/rdep.cu:3721-3731) and nothing tells the other ranks.
"""
from __future__ import annotations

import time
from typing import Optional

import torch.distributed as dist


class PeerLost(RuntimeError):
  pass


class PeerStalled(RuntimeError):
  pass


class Health:
  def __init__(self, rank: int, world: int, store=None, *, stall_s: float = 300.0, prefix: str = "nmoe_health"):
    if store is None:
      if not dist.is_initialized():
        raise RuntimeError("Health needs a store or an initialised process group")
      store = dist.distributed_c10d._get_default_store()
    self.store = dist.PrefixStore(prefix, store)
    self.rank, self.world, self.stall_s = rank, world, stall_s
    self._last_seen = {}          # peer -> (beat payload, local monotonic time when it last changed)
    self.beat(0)

  def beat(self, step: int) -> None:
    try:
      self.store.set(f"hb/{self.rank}", f"{int(step)}")
    except Exception as e:
      raise PeerLost(f"the rendezvous store is unreachable ({type(e).__name__}): the rank that hosts it has left "
                     "the job") from e

  def fail(self, reason: str) -> None:
    """Announce that this rank is leaving the job; never raises (it runs inside exception handlers)."""
    try:
      self.store.set(f"dead/{self.rank}", " ".join(str(reason).split())[:300] or "unknown")
    except Exception:
      pass

  def check(self) -> None:
    try:
      self._check()
    except (PeerLost, PeerStalled):
      raise
    except Exception as e:
      # the store lives in rank 0's process: when it cannot be reached any more, that process is gone
      raise PeerLost(f"the rendezvous store is unreachable ({type(e).__name__}): the rank that hosts it has left "
                     "the job") from e

  def _check(self) -> None:
    now = time.monotonic()
    for r in range(self.world):
      if r == self.rank:
        continue
      if self.store.check([f"dead/{r}"]):
        why = self.store.get(f"dead/{r}").decode(errors="replace")
        raise PeerLost(f"rank {r} left the job: {why}")
      if not self.store.check([f"hb/{r}"]):
        first = self._last_seen.setdefault(r, (None, now))
        if now - first[1] > self.stall_s:
          raise PeerStalled(f"rank {r} never reported in ({self.stall_s:.0f} s)")
        continue
      payload = self.store.get(f"hb/{r}")
      seen = self._last_seen.get(r)
      if seen is None or seen[0] != payload:
        self._last_seen[r] = (payload, now)
      elif now - seen[1] > self.stall_s:
        raise PeerStalled(f"rank {r} has not finished a step for {now - seen[1]:.0f} s "
                          f"(last step {payload.decode(errors='replace')})")


def maybe_health(rank: int, world: int, stall_s: float = 300.0) -> Optional[Health]:
  """A Health object for multi-rank jobs with an initialised process group, else None."""
  if world <= 1 or not dist.is_initialized():
    return None
  return Health(rank, world, stall_s=stall_s)
