"""Executable host model of the RDEP flag / epoch protocol (csrc/rdep.cu), one thread per rank.

The device protocol of one MoE call, per rank:

  plan    write my per-expert counts into row ``rank`` of EVERY peer's count table, then release
          ``count_flags[rank] = epoch`` on every peer; wait (bounded) until all entries of my own count_flags
          reached the epoch; derive -- identically on every rank -- each owner's padded segment layout
  place   store my rows at ``segment start + rows of lower ranks + my stable rank`` in the owner's buffer,
          then release ``data_flags[rank] = data_epoch`` on every peer
  wait    bounded wait on my data_flags; run the experts
  return  store each output row into the SOURCE rank's (token, slot) buffer, release ``ret_flags[rank]``;
          the source waits on its ret_flags and sums the K slots in slot order

This model keeps exactly those tables, flags and epochs in plain Python objects shared between threads, adds random
scheduling jitter, and checks what the kernels rely on but cannot assert cheaply:

* no two rows ever claim the same position of an owner's buffer (deterministic placement, no atomics),
* nobody writes a peer's buffer while its owner is still reading the previous call's rows (the count exchange of
  the next call and the return wait of this call are the only barriers),
* a flag value left over from an earlier epoch never satisfies a later wait,
* when a peer never arrives, every bounded wait of the others runs out, records ``{code, where, peer, epoch}`` like
  ``report_status`` does, and the call returns instead of spinning for ever.

Python's interpreter lock makes every access sequentially consistent, so this model says nothing about memory
ordering (release / acquire scopes); those are argued in the kernel sources.  It is a model of the protocol's logic.
"""
from __future__ import annotations

import random
import threading
import time
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Tuple

WAIT_TIMEOUT = 2          # status codes, as in csrc/common/status.h
WHERE_COUNT, WHERE_DATA, WHERE_RET = 410, 420, 421


@dataclass
class Status:
  code: int = 0
  where: int = 0
  a: int = 0
  b: int = 0

  def report(self, code: int, where: int, a: int, b: int) -> None:
    if self.code == 0:               # first failure wins, like the device record
      self.code, self.where, self.a, self.b = code, where, a, b


@dataclass
class RankMemory:
  """What one rank exposes to its peers."""
  world: int
  n_experts: int
  counts: List[List[int]] = field(default_factory=list)        # [world][E]
  count_flags: List[int] = field(default_factory=list)
  data_flags: List[int] = field(default_factory=list)
  ret_flags: List[int] = field(default_factory=list)
  xbuf: Dict[int, Tuple] = field(default_factory=dict)         # position -> (src rank, pair index, payload)
  ret: Dict[int, float] = field(default_factory=dict)          # pair index -> returned value
  reading: bool = False                                        # owner is consuming xbuf
  violations: List[str] = field(default_factory=list)

  def __post_init__(self):
    self.counts = [[0] * self.n_experts for _ in range(self.world)]
    self.count_flags = [0] * self.world
    self.data_flags = [0] * self.world
    self.ret_flags = [0] * self.world


class Fabric:
  """All ranks' memories plus the jitter source; stands in for NVLink peer access."""

  def __init__(self, world: int, n_experts: int, align: int = 4, seed: int = 0, jitter_s: float = 0.002):
    assert n_experts % world == 0
    self.world, self.E, self.n_local, self.align = world, n_experts, n_experts // world, align
    self.mem = [RankMemory(world, n_experts) for _ in range(world)]
    self.rng = random.Random(seed)
    self.jitter_s = jitter_s
    self.lock = threading.Lock()

  def jitter(self) -> None:
    with self.lock:
      d = self.rng.random() * self.jitter_s
    if d > 0:
      time.sleep(d)


def bounded_wait(flags: List[int], epoch: int, budget_s: float, status: Status, where: int) -> bool:
  """All entries >= epoch before the budget runs out; records the first laggard otherwise."""
  deadline = time.monotonic() + budget_s
  while True:
    lag = [r for r, f in enumerate(flags) if f < epoch]
    if not lag:
      return True
    if time.monotonic() > deadline:
      status.report(WAIT_TIMEOUT, where, lag[0], epoch)
      return False
    time.sleep(0.0005)


class RankActor:
  """One rank's side of the protocol; ``moe_call`` is one forward dispatch -> experts -> return."""

  def __init__(self, fabric: Fabric, rank: int, wait_budget_s: float = 1.0):
    self.f, self.rank, self.budget = fabric, rank, wait_budget_s
    self.status = Status()
    self.epoch_count = self.epoch_data = self.epoch_ret = 0

  # -- plan: count exchange + identical layout on every rank
  def plan(self, eid: List[int]) -> Optional[dict]:
    f, me = self.f, self.f.mem[self.rank]
    mine = [0] * f.E
    local_rank = []
    for e in eid:
      local_rank.append(mine[e])
      mine[e] += 1
    self.epoch_count += 1
    for r in range(f.world):
      f.jitter()
      f.mem[r].counts[self.rank] = list(mine)
    for r in range(f.world):
      f.mem[r].count_flags[self.rank] = self.epoch_count
    if not bounded_wait(me.count_flags, self.epoch_count, self.budget, self.status, WHERE_COUNT):
      return None
    base, seg_start, total_rows = {}, {}, 0
    for owner in range(f.world):
      run = 0
      for le in range(f.n_local):
        e = owner * f.n_local + le
        tot = sum(me.counts[r][e] for r in range(f.world))
        low = sum(me.counts[r][e] for r in range(self.rank))
        base[e] = run + low
        seg_start[e] = run
        run += (tot + f.align - 1) // f.align * f.align
      if owner == self.rank:
        total_rows = run
    return {"eid": eid, "local_rank": local_rank, "base": base, "rows": total_rows}

  def place(self, plan: dict, payload: Callable[[int], float]) -> None:
    f = self.f
    self.epoch_data += 1
    for i, e in enumerate(plan["eid"]):
      owner = e // f.n_local
      pos = plan["base"][e] + plan["local_rank"][i]
      dst = f.mem[owner]
      f.jitter()
      if dst.reading:
        dst.violations.append(f"rank {self.rank} wrote position {pos} of rank {owner} while it was being read")
      prev = dst.xbuf.get(pos)
      if prev is not None and prev[3] == self.epoch_data:
        dst.violations.append(f"position {pos} of rank {owner} claimed twice in epoch {self.epoch_data}")
      dst.xbuf[pos] = (self.rank, i, payload(i), self.epoch_data)
    for r in range(f.world):
      f.mem[r].data_flags[self.rank] = self.epoch_data

  def experts_and_return(self, fn: Callable[[int, float], float]) -> bool:
    f, me = self.f, self.f.mem[self.rank]
    if not bounded_wait(me.data_flags, self.epoch_data, self.budget, self.status, WHERE_DATA):
      return False
    me.reading = True
    rows = [(pos, rec) for pos, rec in me.xbuf.items() if rec[3] == self.epoch_data]
    f.jitter()
    outs = [(src, pair, fn(self.rank, val)) for _pos, (src, pair, val, _ep) in sorted(rows)]
    me.reading = False                    # every reader of the peer-written buffer is done before rows go back
    self.epoch_ret += 1
    for src, pair, y in outs:
      f.jitter()
      f.mem[src].ret[(self.epoch_ret, pair)] = y
    for r in range(f.world):
      f.mem[r].ret_flags[self.rank] = self.epoch_ret
    return True

  def gather(self, n_pairs: int) -> Optional[List[float]]:
    me = self.f.mem[self.rank]
    if not bounded_wait(me.ret_flags, self.epoch_ret, self.budget, self.status, WHERE_RET):
      return None
    return [me.ret.pop((self.epoch_ret, i)) for i in range(n_pairs)]

  def moe_call(self, eid: List[int], payload: Callable[[int], float], fn: Callable[[int, float], float]):
    plan = self.plan(eid)
    if plan is None:
      return None
    self.place(plan, payload)
    if not self.experts_and_return(fn):
      return None
    return self.gather(len(eid))


def run_ranks(world: int, n_experts: int, calls: int, pairs_per_rank: int, *, absent: Tuple[int, ...] = (),
              die_after_counts: Tuple[int, ...] = (), seed: int = 0, wait_budget_s: float = 1.0, align: int = 4):
  """Run ``calls`` consecutive MoE calls on ``world`` rank threads.  Ranks in ``absent`` never start; ranks in
  ``die_after_counts`` publish their counts of the first call and then stop.  Returns (results, statuses,
  violations): results[rank] is the list of per-call outputs (None from the call on which a wait ran out)."""
  fabric = Fabric(world, n_experts, align=align, seed=seed)
  actors = [RankActor(fabric, r, wait_budget_s) for r in range(world)]
  results: List[List] = [[] for _ in range(world)]
  routing = random.Random(seed + 1)
  eids = [[[routing.randrange(n_experts) for _ in range(pairs_per_rank)] for _ in range(world)] for _ in range(calls)]

  def body(r: int):
    a = actors[r]
    for c in range(calls):
      if r in die_after_counts:
        a.plan(eids[c][r])
        return
      out = a.moe_call(eids[c][r], payload=lambda i, r=r, c=c: 1000.0 * c + 10.0 * r + 0.001 * i,
                       fn=lambda owner, v: 2.0 * v + owner)
      results[r].append(out)
      if out is None:
        return

  threads = [threading.Thread(target=body, args=(r,), daemon=True) for r in range(world) if r not in absent]
  for t in threads:
    t.start()
  for t in threads:
    t.join(timeout=30 + 4 * wait_budget_s * calls)
  hung = [t for t in threads if t.is_alive()]
  violations = [v for m in fabric.mem for v in m.violations]
  if hung:
    violations.append(f"{len(hung)} rank thread(s) never returned")
  return results, [a.status for a in actors], violations, eids
