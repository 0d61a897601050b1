"""Deterministic loader: one global stream of sequences, each rank takes its slice.

Every step the loader walks ``batch_size`` selections of the global stream (sources are mixed by
smooth weighted round-robin with integer weights, stages advance when their quotas are spent);
rank r materialises only selections [r*B/W, (r+1)*B/W) and merely advances cursors for the
others, so the stream -- and therefore resume -- does not depend on the world size.  State is a
few integers per source (nmoe/data/loader.py:32-259).

Batches are assembled into a pinned host buffer and copied to the device asynchronously.
``SyntheticLoader`` emits uniform random token ids with the same interface and exact resume.
"""
from __future__ import annotations

import os
from glob import glob
from pathlib import Path
from typing import Dict, List, Optional, Tuple

import numpy as np
import torch

from .dataset import Cursor, NumpyFSLDataset
from .mixture import MixturePlan, populate_paths, resolve_plan, single_source_plan


class _SourceState:
  __slots__ = ("dataset", "cursor", "emitted")

  def __init__(self, dataset: Optional[NumpyFSLDataset]):
    self.dataset, self.cursor, self.emitted = dataset, Cursor(), 0


class _PinnedRing:
  """A few pinned host staging buffers used in turn.  A buffer is rewritten only after the host has waited for the
  event recorded behind the last host->device copy that read it, so an asynchronous copy can never see the next
  step's tokens (or a half-written batch), however far the host runs ahead of the device."""

  def __init__(self, shape, n: int = 3):
    self.cuda = torch.cuda.is_available()
    self.bufs = [torch.empty(*shape, dtype=torch.int64) for _ in range(n)]
    if self.cuda:
      self.bufs = [b.pin_memory() for b in self.bufs]
    self.events = [None] * n
    self.i = -1

  def acquire(self) -> torch.Tensor:
    """Next buffer, safe to overwrite."""
    self.i = (self.i + 1) % len(self.bufs)
    ev = self.events[self.i]
    if ev is not None:
      ev.synchronize()
      self.events[self.i] = None
    return self.bufs[self.i]

  def copied(self, stream=None) -> None:
    """Call right after enqueueing the copy that reads the buffer returned by the last acquire()."""
    if self.cuda:
      ev = torch.cuda.Event()
      ev.record(stream if stream is not None else torch.cuda.current_stream())
      self.events[self.i] = ev

  def to_device(self, buf: torch.Tensor, device: torch.device) -> torch.Tensor:
    if device.type != "cuda":
      return buf.clone()        # the caller must not alias a buffer that will be rewritten
    out = buf.to(device, non_blocking=True)
    self.copied()
    return out


class DeterministicLoader:
  def __init__(self, *, plan: MixturePlan, dp_world_size: int, dp_rank: int, seq_len: int, tokens_per_update: int,
               device: str | torch.device = "cuda"):
    self.plan, self.world, self.rank = plan, int(dp_world_size), int(dp_rank)
    self.seq_len, self.device = int(seq_len), torch.device(device)
    self.seqs_per_step = max(1, int(tokens_per_update) // self.seq_len)
    q, r = divmod(self.seqs_per_step, self.world)
    self.mine = q + (1 if self.rank < r else 0)
    self.start = self.rank * q + min(self.rank, r)
    self.global_seq_idx = 0
    self._stage_index = -1
    self._acc: List[int] = []
    self._wsum = 1
    self._src: Dict[str, _SourceState] = {}
    self._enter_stage(0)
    self._pin: Optional[torch.Tensor] = None
    self._ring: Optional[_PinnedRing] = None

  # ---------------------------------------------------------------- stream mechanics
  def _enter_stage(self, idx: int) -> None:
    self._stage_index = idx
    st = self.plan.stages[idx]
    self._acc = [0] * len(st.sources)
    self._wsum = sum(sp.weight_fp for sp in st.sources) or 1
    self._src = {sp.id: _SourceState(NumpyFSLDataset(sp.paths) if sp.paths else None) for sp in st.sources}

  def _maybe_advance_stage(self) -> None:
    st = self.plan.stages[self._stage_index]
    if all(self._src[sp.id].emitted >= sp.quota_sequences for sp in st.sources) \
        and self._stage_index + 1 < len(self.plan.stages):
      self._enter_stage(self._stage_index + 1)

  def _pick(self) -> int:
    """Smooth weighted round-robin over sources that still have quota."""
    st = self.plan.stages[self._stage_index]
    for _ in range(2 * len(st.sources)):
      for i, sp in enumerate(st.sources):
        self._acc[i] += sp.weight_fp
      k = int(np.argmax(self._acc))
      self._acc[k] -= self._wsum
      sp = st.sources[k]
      if self._src[sp.id].emitted < sp.quota_sequences:
        return k
    raise StopIteration

  def _take(self, k: int, materialise: bool) -> Optional[np.ndarray]:
    sp = self.plan.stages[self._stage_index].sources[k]
    ss = self._src[sp.id]
    if ss.dataset is None:
      raise RuntimeError(f"no shard paths for source '{sp.id}'")
    arr = None
    if materialise:
      arr, ss.cursor = ss.dataset.next_window(ss.cursor, self.seq_len + 1)
    else:
      ss.cursor = ss.dataset.advance(ss.cursor, self.seq_len + 1)
    ss.emitted += 1
    self.global_seq_idx += 1
    return arr

  # ---------------------------------------------------------------- public
  def next_host(self) -> torch.Tensor:
    """This rank's [mine, seq_len+1] int64 batch in pinned host memory.  The buffer is one of a small ring; a
    caller that copies it to the device itself should call ``staging.copied()`` right after enqueueing the copy."""
    if self._ring is None:
      self._ring = _PinnedRing((self.mine, self.seq_len + 1))
    self._pin = self._ring.acquire()
    row = 0
    for i in range(self.seqs_per_step):
      self._maybe_advance_stage()
      k = self._pick()
      arr = self._take(k, self.start <= i < self.start + self.mine)
      if arr is not None:
        self._pin[row].copy_(torch.from_numpy(arr.astype(np.int64)))
        row += 1
    if row == 0:
      raise StopIteration
    return self._pin

  @property
  def staging(self) -> "_PinnedRing":
    return self._ring

  @torch.no_grad()
  def next(self) -> Tuple[torch.Tensor, torch.Tensor]:
    host = self.next_host()
    batch = self._ring.to_device(host, torch.device(self.device))
    return batch[:, :-1], batch[:, 1:]

  def state_dict(self) -> Dict:
    st = self.plan.stages[self._stage_index]
    return {
      "version": 1, "current_stage": st.stage_id, "stage_index": self._stage_index,
      "global_sequence_index": self.global_seq_idx, "accumulators": list(self._acc),
      "emitted_sequences": {sp.id: self._src[sp.id].emitted for sp in st.sources},
      "cursors": {sp.id: dict(vars(self._src[sp.id].cursor)) for sp in st.sources},
    }

  def load_state_dict(self, state: Dict) -> None:
    self._enter_stage(int(state.get("stage_index", 0)))
    self.global_seq_idx = int(state.get("global_sequence_index", 0))
    self._acc = [int(v) for v in state.get("accumulators", self._acc)]
    for sid, n in state.get("emitted_sequences", {}).items():
      if sid in self._src:
        self._src[sid].emitted = int(n)
    for sid, d in state.get("cursors", {}).items():
      if sid in self._src:
        self._src[sid].cursor = Cursor(int(d.get("file_idx", 0)), int(d.get("pos_in_file", 0)),
                                       int(d.get("wrap_count", 0)))

  def close(self) -> None:
    pass


class SyntheticLoader:
  """Uniform random token ids (never the EOS id); the batch of step s depends only on (seed, s, rank)."""

  def __init__(self, *, vocab_size: int, eos_token_id: int, batch_per_rank: int, seq_len: int, rank: int, seed: int,
               device: str | torch.device = "cuda"):
    self.vocab, self.eos = vocab_size, eos_token_id
    self.mine, self.seq_len, self.rank, self.seed = batch_per_rank, seq_len, rank, seed
    self.device = torch.device(device)
    self.step = 0
    self._ring = _PinnedRing((self.mine, seq_len + 1))

  def next_host(self) -> torch.Tensor:
    g = torch.Generator().manual_seed(self.seed * 1_000_003 + self.step * 1009 + self.rank)
    hi = self.vocab - 1 if self.eos == self.vocab - 1 else self.vocab
    t = torch.randint(0, hi, (self.mine, self.seq_len + 1), generator=g)
    if hi == self.vocab:
      t = torch.where(t == self.eos, (t + 1) % self.vocab, t)
    pin = self._ring.acquire()
    pin.copy_(t)
    self.step += 1
    return pin

  @property
  def staging(self) -> "_PinnedRing":
    return self._ring

  def next(self) -> Tuple[torch.Tensor, torch.Tensor]:
    host = self.next_host()
    batch = self._ring.to_device(host, self.device)
    return batch[:, :-1], batch[:, 1:]

  def state_dict(self) -> Dict:
    return {"version": 1, "synthetic": True, "step": self.step}

  def load_state_dict(self, state: Dict) -> None:
    self.step = int(state.get("step", 0))

  def close(self) -> None:
    pass


def preflight(plan: MixturePlan, seq_len: int, print_fn=print, mode: Optional[str] = None) -> None:
  """Compare every source's tokens on disk with its quota.  A short source makes the stream wrap (the same documents
  are seen again): ``mode="warn"`` (default) says so, ``"strict"`` refuses to start, as the reference does
  (nmoe/data/loader.py:286-306), ``"off"`` skips the check.  ``NMOE_PREFLIGHT`` sets the mode from the environment.
  A source without any shard is an error in every mode."""
  mode = (mode or os.environ.get("NMOE_PREFLIGHT", "warn")).lower()
  if mode not in ("warn", "strict", "off"):
    raise ValueError(f"preflight mode {mode!r}: expected warn, strict or off")
  short = []
  for st in plan.stages:
    for sp in st.sources:
      if not sp.paths:
        raise RuntimeError(f"stage {st.stage_id}: source '{sp.id}' has no .npy shards")
      if mode == "off":
        continue
      have = sum(os.path.getsize(p) for p in sp.paths) // 4
      need = sp.quota_sequences * (seq_len + 1)
      if have < need:
        short.append(f"source '{sp.id}' in stage '{st.stage_id}': {have:,} tokens on disk < {need:,} needed")
  if short and mode == "strict":
    raise RuntimeError("preflight failed: " + "; ".join(short) + ".  Check data_root, prepare more data or lower the flow's scale.")
  for line in short:
    print_fn(f"[preflight] {line}; the stream will wrap")


def build_loader(cfg, rank: int, world_size: int, split: str = "train", print_fn=print):
  """(loader, plan).  ``data_path = "synthetic"`` (or no data configured) -> SyntheticLoader;
  ``data_path = <dir>`` -> all ``**/*.npy`` below it as one source; ``flow_mode`` -> mixture plan."""
  device = "cuda" if torch.cuda.is_available() else "cpu"
  per_rank = max(1, cfg.batch_size // max(1, world_size))
  if (cfg.data_path in (None, "synthetic")) and not cfg.flow_mode:
    return SyntheticLoader(vocab_size=cfg.vocab_size, eos_token_id=cfg.eos_token_id, batch_per_rank=per_rank,
                           seq_len=cfg.seq_len, rank=rank, seed=cfg.seed, device=device), None
  if cfg.data_path and not cfg.flow_mode:
    shards = sorted(set(glob(str(Path(cfg.data_path) / "**" / "*.npy"), recursive=True)))
    if not shards:
      raise RuntimeError(f"no .npy shards found under {cfg.data_path}")
    need = cfg.steps * cfg.batch_size * cfg.seq_len
    plan = single_source_plan(shards, cfg.seq_len, need)
    if rank == 0:
      print_fn(f"streaming from {cfg.data_path}: {len(shards)} shards, {need:,} tokens needed")
      preflight(plan, cfg.seq_len, print_fn)
  else:
    if not (cfg.mixture_toml and cfg.flow_profiles_toml):
      raise ValueError("flow_mode needs mixture_toml and flow_profiles_toml")
    plan = resolve_plan(mixture_toml=Path(cfg.mixture_toml), flow_profiles_toml=Path(cfg.flow_profiles_toml),
                        flow_section=f"flow.{cfg.flow_mode}", seq_len=cfg.seq_len, active_params_b=cfg.active_params_b)
    registry = None
    if getattr(cfg, "tasks_toml", None):
      from .registry import Registry
      registry = Registry.load(cfg.tasks_toml)
    populate_paths(plan, dataset_root=Path(cfg.data_root) / "flows" / cfg.flow_mode, split=split, registry=registry)
    missing = [f"{st.stage_id}/{sp.id}" for st in plan.stages for sp in st.sources if not sp.paths]
    if missing:
      where = f"{Path(cfg.data_root) / 'flows' / cfg.flow_mode}" + (f" or as tasks of {cfg.tasks_toml}" if registry is not None else "")
      raise RuntimeError(f"sources without shards (not ready): {', '.join(missing)}; looked under {where}.  "
                         "Build them with `data.cli prep-mixture` or `data.cli prep --task ID`.")
    flow_tokens = int(sum(s.total_tokens_b for s in plan.stages) * 1e9)
    if cfg.steps <= 0:
      cfg.steps = flow_tokens // (cfg.batch_size * cfg.seq_len)
    if rank == 0:
      preflight(plan, cfg.seq_len, print_fn)
  loader = DeterministicLoader(plan=plan, dp_world_size=world_size, dp_rank=rank, seq_len=cfg.seq_len,
                               tokens_per_update=cfg.batch_size * cfg.seq_len, device=device)
  return loader, plan
