"""Stopping a training job on request: checkpoint at a step every rank agrees on, then leave.

A scheduler that preempts a job sends SIGTERM and kills it a grace period later; an operator may want the same effect
by hand (SIGUSR1).  Dying in mid-step loses the work since the last checkpoint and, in a multi-rank job, leaves the
other ranks waiting in collectives.  ``StopRequest`` turns the signal into a flag that the training loop looks at
between steps:

* one rank: stop after the current step;
* several ranks: the signal reaches the ranks at slightly different times, possibly one step apart.  The first rank to
  see it proposes ``stop_at = its step + margin`` through the rendezvous store (compare-and-set: the first proposal
  stands); every rank reads that key between steps and stops when it reaches the step.  Ranks of one job are never
  more than a step apart (each step's collectives keep them together), so with ``margin = 2`` every rank learns of the
  stop before it gets there, and all of them checkpoint the same step.

A second signal is not intercepted: it acts as it would have without this module (so a launcher that tears a job
down is never kept waiting by a rank stuck in a collective).

The training loop then writes a checkpoint for that step, records the run as ``killed`` and returns; a restart with the
same configuration resumes from it exactly.  The reference has no counterpart (its runs end as ``completed`` or
``failed``; the ``killed`` status exists in its schema but nothing sets it, nmoe/experiments.py:150-163).
"""
from __future__ import annotations

import os
import signal
from typing import Iterable, Optional

import torch.distributed as dist


class StopRequest:
  KEY = "stop_at"

  def __init__(self, world: int = 1, store=None, *, margin: int = 2, signals: Iterable[int] = (signal.SIGTERM, signal.SIGUSR1),
               install: bool = True, prefix: str = "nmoe_stop"):
    self.world, self.margin = int(world), int(margin)
    self.requested = False            # set by the signal handler (or by request())
    self.reason = ""
    self.stop_at: Optional[int] = None
    self._old = {}
    self.store = None
    if self.world > 1:
      if store is None:
        if not dist.is_initialized():
          raise RuntimeError("StopRequest for several ranks needs a store or an initialised process group")
        store = dist.distributed_c10d._get_default_store()
      self.store = dist.PrefixStore(prefix, store)
    if install:
      for s in signals:
        try:
          self._old[s] = signal.signal(s, self._on_signal)
        except (ValueError, OSError):      # not the main thread, or a signal this platform lacks
          pass

  def _on_signal(self, signum, _frame) -> None:
    # nothing but a flag here: the handler can run in the middle of anything
    if self.requested:
      # asked twice: the sender is not waiting for a checkpoint (a launcher tearing the job down after another rank
      # failed, an impatient operator).  Put the original disposition back and let the signal do what it would have done.
      self.restore()
      os.kill(os.getpid(), signum)
      return
    self.requested = True
    self.reason = signal.Signals(signum).name

  def request(self, reason: str = "requested") -> None:
    self.requested, self.reason = True, reason

  def restore(self) -> None:
    for s, h in self._old.items():
      try:
        signal.signal(s, h)
      except (ValueError, OSError):
        pass
    self._old = {}

  def should_stop(self, step: int) -> bool:
    """Call after step ``step`` has finished (1-based, the same number on every rank for the same step).  True exactly
    once per rank, at the agreed step."""
    if self.world <= 1:
      if self.requested and self.stop_at is None:
        self.stop_at = step
      return self.stop_at is not None and step >= self.stop_at
    if self.stop_at is None:
      try:
        if self.requested:
          # first proposal wins; the call returns whatever is stored afterwards
          got = self.store.compare_set(self.KEY, "", str(step + self.margin))
          self.stop_at = int(got.decode() if isinstance(got, (bytes, bytearray)) else got)
        elif self.store.check([self.KEY]):
          self.stop_at = int(self.store.get(self.KEY).decode())
      except Exception:
        # the store's host is gone: the job is ending anyway, and the liveness check reports it; do not stop on a guess
        return False
    return self.stop_at is not None and step >= self.stop_at
