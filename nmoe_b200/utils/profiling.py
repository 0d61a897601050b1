"""Step profiling with ``torch.profiler``, driven by the ``profiling_*`` configuration keys, and named scopes for it.

``profiling_enabled = true`` makes the training loop record ``profiling_steps`` steps (after ``profiling_skip`` steps of
the run and one warm-up step of the profiler) and write, per rank, into ``profiling_output_dir/{run}``:

  trace_rank{r}.json   a Chrome / Perfetto trace (CPU ops, CUDA kernels when there is a GPU, the scopes below)
  ops_rank{r}.txt      the operator table sorted by device time (host time on a CPU)

Scopes (``embed``, ``block_NN/attn``, ``block_NN/ffn``, ``final_norm``, ``lm_head_loss``, ``backward``, ``optimizer``)
are ``torch.profiler.record_function`` ranges (nmoe/model.py:46-268 puts one on every module).  They are switched on
only while a profile is being taken: outside of it ``scope()`` hands back one shared do-nothing context, so the
training loop pays an attribute read per scope and nothing else.

This is a host-side tool.  Kernel counters come from ``ncu`` on one small case per kernel (see ``profiles/``); a
number measured under any profiler is never a benchmark figure.
"""
from __future__ import annotations

from contextlib import nullcontext
from pathlib import Path
from typing import Callable, Optional

import torch

_OFF = nullcontext()
_enabled = False


def scopes_enabled() -> bool:
  return _enabled


def enable_scopes(on: bool = True) -> None:
  global _enabled
  _enabled = bool(on)


def scope(name: str):
  """``with scope("block_03/attn"):`` -- a profiler range while a profile is being taken, nothing otherwise."""
  return torch.profiler.record_function(name) if _enabled else _OFF


class StepProfiler:
  """Call ``step()`` once at the end of every training step; everything else happens inside.  ``done`` turns true when
  the files are written.  A profiler that is never enabled costs one comparison per step."""

  def __init__(self, enabled: bool, out_dir, rank: int = 0, *, steps: int = 10, skip: int = 2, print_fn: Callable = print,
               with_stack: bool = False):
    self.enabled, self.rank, self.steps, self.skip, self.print = bool(enabled) and steps > 0, rank, int(steps), max(0, int(skip)), print_fn
    self.dir = Path(out_dir)
    self.with_stack = with_stack
    self._prof: Optional[torch.profiler.profile] = None
    self._seen = 0
    self.done = not self.enabled
    self.files: list = []

  def _start(self) -> None:
    acts = [torch.profiler.ProfilerActivity.CPU]
    if torch.cuda.is_available():
      acts.append(torch.profiler.ProfilerActivity.CUDA)
    self._prof = torch.profiler.profile(activities=acts, record_shapes=False, with_stack=self.with_stack,
                                        schedule=torch.profiler.schedule(wait=0, warmup=1, active=self.steps, repeat=1))
    enable_scopes(True)
    self._prof.__enter__()

  def _finish(self) -> None:
    prof, self._prof = self._prof, None
    prof.__exit__(None, None, None)
    enable_scopes(False)
    self.dir.mkdir(parents=True, exist_ok=True)
    trace, table = self.dir / f"trace_rank{self.rank}.json", self.dir / f"ops_rank{self.rank}.txt"
    prof.export_chrome_trace(str(trace))
    key = "self_cuda_time_total" if torch.cuda.is_available() else "self_cpu_time_total"
    try:
      text = prof.key_averages().table(sort_by=key, row_limit=60)
    except Exception:                # sort keys were renamed between torch versions; the unsorted table still helps
      text = prof.key_averages().table(row_limit=60)
    table.write_text(text)
    self.files = [trace, table]
    self.done = True
    self.print(f"[profile] rank {self.rank}: {self.steps} step(s) -> {trace} and {table.name}")

  def step(self) -> None:
    if self.done:
      return
    self._seen += 1
    if self._prof is None:
      if self._seen > self.skip:
        self._start()                # the next step is the profiler's warm-up step
      return
    self._prof.step()
    if self._seen > self.skip + 1 + self.steps:
      self._finish()

  def close(self) -> None:
    """End of training before the profile was complete: write what there is."""
    if self._prof is not None:
      self._finish()
