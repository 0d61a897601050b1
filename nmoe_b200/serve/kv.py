"""Paged KV-cache bookkeeping with prefix sharing (host side; the tensors live in the engine).

A sequence owns a *block table*: the list of cache blocks (``block_size`` token slots each) that
hold its keys/values in order.  Full blocks are content-addressed by a hash chained over the whole
prefix, so two requests that start with the same tokens (a shared grading rubric, a few-shot
header) map their leading blocks to the same physical block and only the first one computes them.

Behavioural counterpart: ``BlockManager`` in the reference engine (nmoe/data/model.py:65-139).
Differences: a freed block keeps its hash until it is re-used (a later request with the same
prefix can still revive it), and the hash is ``blake2b`` from the standard library.
"""
from __future__ import annotations

import hashlib
import itertools
from collections import OrderedDict
from dataclasses import dataclass, field
from enum import IntEnum
from typing import Dict, List, Optional, Sequence as Seq

import numpy as np


class SeqStatus(IntEnum):
  WAITING = 0
  RUNNING = 1
  FINISHED = 2


_ids = itertools.count(1)


@dataclass
class Sequence:
  tokens: List[int]
  max_new_tokens: int = 256
  seq_id: int = field(default_factory=lambda: next(_ids))
  status: SeqStatus = SeqStatus.WAITING
  block_table: List[int] = field(default_factory=list)
  n_cached: int = 0                 # leading tokens whose K/V were found in the prefix cache
  prompt_len: int = 0

  def __post_init__(self):
    self.tokens = list(self.tokens)
    self.prompt_len = self.prompt_len or len(self.tokens)

  def __len__(self) -> int:
    return len(self.tokens)

  @property
  def n_generated(self) -> int:
    return len(self.tokens) - self.prompt_len


class BlockPool:
  """Reference-counted pool of ``num_blocks`` cache blocks with a content-addressed prefix cache."""

  def __init__(self, num_blocks: int, block_size: int = 16):
    self.block_size = block_size
    self.num_blocks = num_blocks
    self.ref = [0] * num_blocks
    self.hash_of: List[Optional[bytes]] = [None] * num_blocks
    self.ready = [False] * num_blocks          # K/V of the block have been written (set by the engine after prefill)
    self.by_hash: Dict[bytes, int] = {}
    # free blocks in LRU order; blocks that still carry a hash sit at the end so that plain
    # blocks are recycled first and cached prefixes survive as long as possible
    self.free: "OrderedDict[int, None]" = OrderedDict((i, None) for i in range(num_blocks))
    self.hits = 0
    self.misses = 0

  # ------------------------------------------------------------------ helpers
  def blocks_for(self, n_tokens: int) -> int:
    return (n_tokens + self.block_size - 1) // self.block_size

  @staticmethod
  def _chain(prev: Optional[bytes], tokens: Seq[int]) -> bytes:
    h = hashlib.blake2b(digest_size=16)
    if prev is not None:
      h.update(prev)
    h.update(np.asarray(tokens, dtype=np.int32).tobytes())
    return h.digest()

  def _take(self, prefer: Optional[int] = None) -> int:
    if prefer is not None:
      self.free.pop(prefer)
      return prefer
    if not self.free:
      raise RuntimeError("KV cache exhausted")
    bid, _ = self.free.popitem(last=False)
    old = self.hash_of[bid]
    if old is not None and self.by_hash.get(old) == bid:
      del self.by_hash[old]
    self.hash_of[bid] = None
    self.ready[bid] = False
    return bid

  @property
  def n_free(self) -> int:
    return len(self.free)

  # ------------------------------------------------------------------ prompt admission
  def can_allocate(self, seq: Sequence) -> bool:
    return self.n_free >= self.blocks_for(len(seq)) - len(seq.block_table)

  def allocate(self, seq: Sequence) -> None:
    """Give ``seq`` blocks for all its current tokens; leading full blocks found in the prefix
    cache are shared and counted in ``seq.n_cached`` (the engine skips their prefill).  The last
    token is never served from the cache: its logits are needed."""
    bs = self.block_size
    n_blocks = self.blocks_for(len(seq))
    prev: Optional[bytes] = None
    sharing = len(seq.block_table) == 0
    for i in range(len(seq.block_table), n_blocks):
      chunk = seq.tokens[i * bs:(i + 1) * bs]
      full = len(chunk) == bs
      h = self._chain(prev, chunk) if full else None
      bid = self.by_hash.get(h) if (full and sharing) else None
      if bid is not None and self.ready[bid] and (i + 1) * bs < len(seq):
        if self.ref[bid] == 0:
          self._take(bid)                      # revive a freed block whose content is still valid
        self.ref[bid] += 1
        seq.block_table.append(bid)
        seq.n_cached = (i + 1) * bs
        self.hits += 1
      else:
        sharing = False
        bid = self._take()
        self.ref[bid] = 1
        if h is not None:
          self.misses += 1
          known = self.by_hash.get(h)
          if known is None or not self.ready[known]:       # keep an existing, already written copy addressable
            self.by_hash[h] = bid
            self.hash_of[bid] = h
        seq.block_table.append(bid)
      prev = h

  def mark_ready(self, seq: Sequence) -> None:
    """The K/V of every block of ``seq`` are in the cache: later requests may share them."""
    for bid in seq.block_table:
      self.ready[bid] = True

  # ------------------------------------------------------------------ decode
  def can_append(self, seq: Sequence) -> bool:
    return (len(seq) - 1) // self.block_size < len(seq.block_table) or self.n_free > 0

  def append_slot(self, seq: Sequence) -> int:
    """Cache slot of ``seq``'s last token (allocating a fresh block at a block boundary)."""
    pos = len(seq) - 1
    bi = pos // self.block_size
    if bi >= len(seq.block_table):
      bid = self._take()
      self.ref[bid] = 1
      seq.block_table.append(bid)
    return seq.block_table[bi] * self.block_size + pos % self.block_size

  def slot(self, seq: Sequence, pos: int) -> int:
    return seq.block_table[pos // self.block_size] * self.block_size + pos % self.block_size

  # ------------------------------------------------------------------ release
  def release(self, seq: Sequence) -> None:
    for bid in seq.block_table:
      self.ref[bid] -= 1
      if self.ref[bid] == 0:
        self.free[bid] = None
        if self.hash_of[bid] is None:
          self.free.move_to_end(bid, last=False)     # plain blocks are recycled before cached prefixes
    seq.block_table = []
    seq.n_cached = 0
