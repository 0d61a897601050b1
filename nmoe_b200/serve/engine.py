"""Continuous-batching inference engine over the paged KV cache.

  eng = Engine(model, max_seq_len=4096, max_batch=128)
  sid = eng.add(prompt_tokens, max_new_tokens=64)
  while not eng.idle:
      logits, ids = eng.step()            # one prefill batch or one decode step
      for row, sid in zip(logits, ids):
          tok = int(row.argmax())
          eng.update(sid, tok, finished=tok in stop_tokens)

Each ``step`` either admits waiting requests (as many as fit in the batch and in the cache; their
prompts are prefilled together, minus any prefix already in the cache) or advances every running
sequence by one token.  ``generate`` wraps the loop for greedy / top-k sampling; ``hidden_states``
runs prompts through the first layers only (the probe / judge taps of the curation stack).

Behavioural counterpart: ``BatchedGenerator`` (nmoe/data/model.py:650-790).  Differences: prefix
blocks found in the cache are really attended to during prefill, the host-side batch assembly is
vectorised, and a request that cannot get a cache block is preempted back to the queue instead of
raising.
"""
from __future__ import annotations

from collections import deque
from typing import Callable, Deque, Dict, Iterable, List, Optional, Sequence as Seq, Tuple

import torch

from .kv import BlockPool, SeqStatus, Sequence
from .model import CacheView, Transformer


class Engine:
  def __init__(self, model: Transformer, *, max_seq_len: int = 512, max_batch: int = 32, block_size: int = 16,
               num_blocks: Optional[int] = None, max_prefill_tokens: int = 16384):
    self.model = model
    cfg = model.cfg
    self.device = model.embed.device
    self.max_seq_len, self.max_batch, self.block_size = max_seq_len, max_batch, block_size
    self.max_prefill_tokens = max_prefill_tokens
    per_seq = (max_seq_len + block_size - 1) // block_size
    self.num_blocks = num_blocks or max_batch * per_seq
    shape = (cfg.num_hidden_layers, self.num_blocks, block_size, cfg.num_key_value_heads, cfg.head_dim)
    self.k_cache = torch.zeros(shape, dtype=model.embed.dtype, device=self.device)
    self.v_cache = torch.zeros(shape, dtype=model.embed.dtype, device=self.device)
    self.pool = BlockPool(self.num_blocks, block_size)
    self.waiting: Deque[Sequence] = deque()
    self.running: List[Sequence] = []
    self.finished: Dict[int, Sequence] = {}
    self.steps = {"prefill": 0, "decode": 0, "prefill_tokens": 0, "cached_tokens": 0, "preempted": 0}

  # ------------------------------------------------------------------ requests
  def add(self, tokens: Seq[int], max_new_tokens: Optional[int] = None) -> int:
    if len(tokens) == 0 or len(tokens) >= self.max_seq_len:
      raise ValueError(f"prompt length {len(tokens)} outside (0, {self.max_seq_len})")
    seq = Sequence(list(tokens), max_new_tokens or (self.max_seq_len - len(tokens)))
    self.waiting.append(seq)
    return seq.seq_id

  @property
  def idle(self) -> bool:
    return not self.waiting and not self.running

  # ------------------------------------------------------------------ scheduling
  def _admit(self) -> List[Sequence]:
    batch: List[Sequence] = []
    budget = self.max_prefill_tokens
    while self.waiting and len(self.running) + len(batch) < self.max_batch:
      seq = self.waiting[0]
      if not self.pool.can_allocate(seq) or (batch and len(seq) > budget):
        break
      self.waiting.popleft()
      self.pool.allocate(seq)
      seq.status = SeqStatus.RUNNING
      budget -= len(seq) - seq.n_cached
      batch.append(seq)
    return batch

  def _preempt_for_space(self) -> None:
    """Decode needs a fresh block for some sequence and none is free: push the youngest running
    sequences back to the queue (their blocks are released; they prefill again later)."""
    def need() -> int:
      return sum(1 for s in self.running if (len(s) - 1) // self.block_size >= len(s.block_table))
    while len(self.running) > 1 and need() > self.pool.n_free:
      victim = self.running.pop()
      self.pool.release(victim)
      victim.status = SeqStatus.WAITING
      self.waiting.appendleft(victim)
      self.steps["preempted"] += 1

  # ------------------------------------------------------------------ one step
  @torch.inference_mode()
  def step(self, **model_kw) -> Optional[Tuple[torch.Tensor, List[int]]]:
    """Returns (next-token logits [n, vocab] fp32, sequence ids) or None when idle."""
    batch = self._admit()
    if batch:
      self.running.extend(batch)
      return self._prefill(batch, **model_kw), [s.seq_id for s in batch]
    if not self.running:
      return None
    self._preempt_for_space()
    if not self.running:
      return None
    return self._decode(self.running), [s.seq_id for s in self.running]

  def _prefill(self, seqs: List[Sequence], **model_kw) -> torch.Tensor:
    bs = self.block_size
    new = [len(s) - s.n_cached for s in seqs]
    S = max(new)
    B = len(seqs)
    ids = torch.zeros(B, S, dtype=torch.long)
    pos = torch.zeros(B, S, dtype=torch.long)
    slots = torch.full((B, S), -1, dtype=torch.int32)
    max_blocks = max(len(s.block_table) for s in seqs)
    tables = torch.zeros(B, max_blocks, dtype=torch.int32)
    for i, s in enumerate(seqs):
      n, c = new[i], s.n_cached
      ids[i, :n] = torch.tensor(s.tokens[c:], dtype=torch.long)
      p = torch.arange(c, c + n)
      pos[i, :n] = p
      bt = torch.tensor(s.block_table, dtype=torch.long)
      tables[i, :len(s.block_table)] = bt.int()
      slots[i, :n] = (bt[p // bs] * bs + p % bs).int()
    dev = self.device
    cache = CacheView(self.k_cache, self.v_cache, slots.to(dev), block_tables=tables.to(dev),
                      prefix_lens=[s.n_cached for s in seqs], block_size=bs)
    out = self.model(ids.to(dev), pos.to(dev), cache=cache, is_prefill=True, **model_kw)
    for s in seqs:
      self.pool.mark_ready(s)
    self.steps["prefill"] += 1
    self.steps["prefill_tokens"] += sum(new)
    self.steps["cached_tokens"] += sum(s.n_cached for s in seqs)
    if isinstance(out, tuple) or out is None:
      return out
    last = torch.tensor([n - 1 for n in new], device=dev)
    return out[torch.arange(B, device=dev), last]

  def _decode(self, seqs: List[Sequence]) -> torch.Tensor:
    dev = self.device
    slots = torch.tensor([self.pool.append_slot(s) for s in seqs], dtype=torch.int32)
    ids = torch.tensor([s.tokens[-1] for s in seqs], dtype=torch.long)
    pos = torch.tensor([len(s) - 1 for s in seqs], dtype=torch.long)
    ctx = torch.tensor([len(s) for s in seqs], dtype=torch.int32)
    max_blocks = max(len(s.block_table) for s in seqs)
    tables = torch.zeros(len(seqs), max_blocks, dtype=torch.int32)
    for i, s in enumerate(seqs):
      tables[i, :len(s.block_table)] = torch.tensor(s.block_table, dtype=torch.int32)
    cache = CacheView(self.k_cache, self.v_cache, slots.to(dev), block_tables=tables.to(dev), context_lens=ctx.to(dev),
                      block_size=self.block_size)
    self.steps["decode"] += 1
    return self.model(ids.to(dev), pos.to(dev), cache=cache, is_prefill=False)

  def update(self, seq_id: int, token: int, finished: bool = False) -> None:
    for i, s in enumerate(self.running):
      if s.seq_id == seq_id:
        if not finished:
          s.tokens.append(int(token))
        if finished or s.n_generated >= s.max_new_tokens or len(s) >= self.max_seq_len:
          s.status = SeqStatus.FINISHED
          self.pool.release(s)
          self.running.pop(i)
          self.finished[s.seq_id] = s
        return
    raise KeyError(f"sequence {seq_id} is not running")

  # ------------------------------------------------------------------ conveniences
  def generate(self, prompts: Iterable[Seq[int]], *, max_new_tokens: int = 64, stop_tokens: Iterable[int] = (),
               temperature: float = 0.0, top_k: int = 0, generator: Optional[torch.Generator] = None,
               on_token: Optional[Callable[[int, int], None]] = None) -> List[List[int]]:
    """Greedy (temperature 0) or top-k sampled completions, in the order of ``prompts``."""
    stop = set(int(t) for t in stop_tokens)
    order = [self.add(p, max_new_tokens) for p in prompts]
    while not self.idle:
      res = self.step()
      if res is None:
        break
      logits, ids = res
      if temperature <= 0:
        nxt = logits.argmax(-1)
      else:
        lg = logits / temperature
        if top_k > 0:
          kth = lg.topk(min(top_k, lg.size(-1)), dim=-1).values[:, -1:]
          lg = lg.masked_fill(lg < kth, float("-inf"))
        nxt = torch.multinomial(torch.softmax(lg, -1), 1, generator=generator).squeeze(-1)
      for sid, tok in zip(ids, nxt.tolist()):
        if on_token is not None:
          on_token(sid, tok)
        self.update(sid, tok, finished=tok in stop)
    return [self.finished[sid].tokens[self.finished[sid].prompt_len:] for sid in order]

  @torch.inference_mode()
  def hidden_states(self, prompts: List[Seq[int]], up_to_layer: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Hidden states after ``up_to_layer`` blocks for a batch of prompts, without touching the cache:
    (hidden [B,S,H], mask [B,S])."""
    S = max(len(p) for p in prompts)
    ids = torch.zeros(len(prompts), S, dtype=torch.long)
    mask = torch.zeros(len(prompts), S, dtype=torch.bool)
    for i, p in enumerate(prompts):
      ids[i, :len(p)] = torch.tensor(list(p), dtype=torch.long)
      mask[i, :len(p)] = True
    pos = torch.arange(S).expand(len(prompts), S)
    _, taps = self.model(ids.to(self.device), pos.to(self.device), is_prefill=True, up_to_layer=up_to_layer,
                         return_hidden_states=True, no_logits=True)
    return taps[up_to_layer], mask.to(self.device)
