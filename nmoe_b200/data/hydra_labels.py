"""Training data for the quality heads: labelled documents from tables, oracle labels over shards, ranking pairs.

Three kinds of supervision feed ``hydra.train_heads`` (nmoe/data/hydra_dataset.py:28-206, nmoe/data/train.py:228-330):

  * weak signals that ship with web corpora as table columns (fastText quality scores, a language score, taxonomy
    codes for extraction artifacts / missing content): regression and classification targets for the probe (phase A);
  * oracle rubric labels, one JSON line per document named by a shard reference (``docid.SpanRef``): the tokens are
    read straight from the shard (phase B);
  * an ordinal grade per document (FineWeb-Edu's 0..5 ``int_score``): pairs (better, worse) of similar length for the
    judge's ranking term (phase B).

Everything is table-driven here: a ``FieldMap`` says which (possibly nested) column feeds which target, so a new corpus
is a new map rather than a new class; parquet and JSON-lines files go through the same row reader; the pair sampler
keeps one reservoir per (length bucket, grade) cell and picks among the *feasible* grade combinations directly, so it
never loops on rejection.  ``probe_batches`` / ``judge_batches`` assemble the batch dictionaries ``train_heads`` reads.
"""
from __future__ import annotations

import glob as _glob
import json
import math
import random
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Callable, Dict, Iterable, Iterator, List, Optional, Sequence, Tuple

import torch

from .docid import SpanReader, SpanRef
from .hydra import PROBE_TASKS, RUBRIC

DOMAINS: Dict[str, int] = {"web": 0, "code": 1, "science": 2, "math": 3}
LENGTH_EDGES: Tuple[int, ...] = (256, 512, 1024, 2048)      # token-count cut points: 5 buckets, the last open-ended
N_GRADES = 6                                                 # ordinal grades 0..5


@dataclass
class Labelled:
  """One document with whatever supervision its source carries.  ``text`` or ``tokens`` is set, not both needed."""
  domain: str = "web"
  text: Optional[str] = None
  tokens: Optional[List[int]] = None
  signals: Dict[str, float] = field(default_factory=dict)     # probe regression targets by task name
  classes: Dict[str, int] = field(default_factory=dict)       # probe classification targets by task name
  rubric: Optional[Tuple[float, ...]] = None                  # oracle scores in RUBRIC order, each 0..4
  grade: Optional[int] = None                                 # ordinal quality grade 0..5
  n_tokens: Optional[int] = None
  ref: Optional[str] = None

  def ids(self, encode: Callable[[str], List[int]], max_ctx: int) -> List[int]:
    return (self.tokens if self.tokens is not None else encode(self.text or ""))[:max_ctx]


def dig(row: Any, path: str) -> Any:
  """``row["a"]["b"]["c"]`` for ``"a.b.c"``; None as soon as a level is missing or not a mapping."""
  for key in path.split("."):
    if not isinstance(row, dict):
      return None
    row = row.get(key)
  return row


def _num(v: Any) -> Optional[float]:
  try:
    f = float(v)
  except (TypeError, ValueError):
    return None
  return f if math.isfinite(f) else None


@dataclass(frozen=True)
class FieldMap:
  """Which column feeds which target.  Paths are dotted; a missing value leaves the target unset (masked in the loss)."""
  text: str = "text"
  signals: Tuple[Tuple[str, str], ...] = ()          # (probe task, column path) -> float
  classes: Tuple[Tuple[str, str], ...] = ()          # (probe task, column path) -> int class id
  grade: Optional[str] = None
  n_tokens: Optional[str] = None
  require: Tuple[Tuple[str, float], ...] = ()        # (column path, minimum): rows below (or without it) are skipped


EAI_FIELDS = FieldMap(
  signals=(("fasttext_dclm", "quality_signals.fasttext.dclm"),
           ("fasttext_edu", "quality_signals.fasttext.fineweb_edu_approx"),
           ("fasttext_code", "quality_signals.fasttext.eai_web_code"),
           ("fasttext_math", "quality_signals.fasttext.eai_general_math"),
           ("lang_score", "quality_signals.fasttext.english")),
  classes=(("extraction_artifacts", "eai_taxonomy.extraction_artifacts.primary.code"),
           ("missing_content", "eai_taxonomy.missing_content.primary.code")))

FINEWEB_EDU_FIELDS = FieldMap(signals=(("lang_score", "language_score"),), grade="int_score", n_tokens="token_count",
                              require=(("language_score", 0.9),))

FIELD_MAPS: Dict[str, FieldMap] = {"eai": EAI_FIELDS, "fineweb_edu": FINEWEB_EDU_FIELDS}


def _expand(paths) -> List[Path]:
  if isinstance(paths, (str, Path)):
    paths = [paths]
  out: List[Path] = []
  for p in paths:
    p = str(p)
    hits = sorted(_glob.glob(p, recursive=True)) if any(c in p for c in "*?[") else [p]
    out.extend(Path(h) for h in hits)
  return out


def iter_rows(path: Path, batch_rows: int = 1024) -> Iterator[dict]:
  """Rows of a parquet file (nested structs arrive as dicts) or of a JSON-lines file."""
  if path.suffix == ".parquet":
    import pyarrow.parquet as pq
    for batch in pq.ParquetFile(str(path)).iter_batches(batch_size=batch_rows):
      yield from batch.to_pylist()
  else:
    with open(path, encoding="utf-8") as f:
      for line in f:
        if line.strip():
          yield json.loads(line)


class TableLabels:
  """Labelled documents from parquet / JSON-lines files under a ``FieldMap``.  Re-iterable (each pass re-reads)."""

  def __init__(self, paths, fields: FieldMap, domain: str = "web", max_ctx: int = 4096, chars_per_token: int = 4):
    if domain not in DOMAINS:
      raise ValueError(f"unknown domain {domain!r}; one of {sorted(DOMAINS)}")
    self.paths, self.fields, self.domain = _expand(paths), fields, domain
    self.max_chars = max_ctx * chars_per_token      # the tokeniser never sees more text than the context can hold
    if not self.paths:
      raise FileNotFoundError(f"no label files match {paths!r}")

  def __iter__(self) -> Iterator[Labelled]:
    fm = self.fields
    for path in self.paths:
      for row in iter_rows(path):
        text = dig(row, fm.text)
        if not text or not isinstance(text, str):
          continue
        if any((lambda v: v is None or v < lo)(_num(dig(row, col))) for col, lo in fm.require):
          continue
        s = Labelled(domain=self.domain, text=text[:self.max_chars])
        for task, col in fm.signals:
          v = _num(dig(row, col))
          if v is not None:
            s.signals[task] = v
        for task, col in fm.classes:
          v = _num(dig(row, col))
          if v is not None and 0 <= int(v) < PROBE_TASKS[task][0]:
            s.classes[task] = int(v)
        if fm.grade:
          g = _num(dig(row, fm.grade))
          s.grade = int(g) if g is not None and 0 <= int(g) < N_GRADES else None
        if fm.n_tokens:
          n = _num(dig(row, fm.n_tokens))
          s.n_tokens = int(n) if n is not None else None
        yield s


class OracleLabels:
  """Rubric labels joined with shard tokens: lines ``{"doc_id": <shard reference>, "scores": {dim: 0..4}}``.  Lines
  without all five scores, with an unreadable reference, or marked ``"ok": false`` are counted in ``skipped``."""

  def __init__(self, labels_jsonl, data_root, max_ctx: int = 4096, eos_token_id: Optional[int] = None):
    self.path, self.reader, self.max_ctx, self.eos = Path(labels_jsonl), SpanReader(data_root), max_ctx, eos_token_id
    self.skipped = 0

  def __iter__(self) -> Iterator[Labelled]:
    for row in iter_rows(self.path):
      scores = row.get("scores") or {}
      vals = [_num(scores.get(d)) for d in RUBRIC]
      if row.get("ok") is False or any(v is None for v in vals):
        self.skipped += 1
        continue
      try:
        ref = SpanRef.parse(str(row.get("doc_id", "")))
        toks = self.reader.tokens(ref, self.max_ctx, drop_eos=self.eos)
      except (ValueError, OSError):
        self.skipped += 1
        continue
      if toks:
        dom = ref.source if ref.source in DOMAINS else row.get("domain", "web")
        yield Labelled(domain=dom if dom in DOMAINS else "web", tokens=toks, n_tokens=len(toks), ref=str(ref),
                       rubric=tuple(min(4.0, max(0.0, v)) for v in vals))


def length_bucket(n_tokens: Optional[int]) -> int:
  """Bucket of a token count; an unknown length goes to the middle bucket."""
  if n_tokens is None:
    return len(LENGTH_EDGES) // 2
  return sum(1 for e in LENGTH_EDGES if n_tokens >= e)


class GradedPairs:
  """(better, worse) pairs of graded documents of similar length.

  A reservoir of at most ``cell_cap`` documents is kept per (length bucket, grade); replacement follows Algorithm R with
  the cell's own arrival count, so every document that passed through a cell is equally likely to be in it.  A pair is
  drawn by listing the grade combinations (hi, lo) that are *possible* in the bucket right now with ``hi - lo >=
  min_gap`` and picking one; when none exists the gap falls back to ``relaxed_gap``, but relaxed pairs are held to
  ``max_relaxed_frac`` of all pairs issued: past that share the sampler reads more of the stream instead, until
  the stream has been seen twice over, or ``draw_budget`` documents read, without a wider gap turning up."""

  def __init__(self, stream: Iterable[Labelled], min_gap: int = 2, relaxed_gap: int = 1, max_relaxed_frac: float = 0.2,
               cell_cap: int = 256, warm: int = 8, seed: int = 0, draw_budget: int = 4096):
    self._src, self._it = stream, iter(stream)
    self.min_gap, self.relaxed_gap, self.max_relaxed_frac, self.cap, self.warm = min_gap, relaxed_gap, max_relaxed_frac, cell_cap, warm
    self.rng = random.Random(seed)
    nb = len(LENGTH_EDGES) + 1
    self.cells: List[List[List[Labelled]]] = [[[] for _ in range(N_GRADES)] for _ in range(nb)]
    self.arrived = [[0] * N_GRADES for _ in range(nb)]
    self.issued = self.relaxed = self.passes = 0
    self.draw_budget = draw_budget                    # documents one draw may read before it settles for less
    self._barren: Dict[int, int] = {}

  # -- intake
  def add(self, s: Labelled) -> None:
    if s.grade is None or not 0 <= s.grade < N_GRADES:
      return
    b = length_bucket(s.n_tokens)
    cell = self.cells[b][s.grade]
    self.arrived[b][s.grade] += 1
    if len(cell) < self.cap:
      cell.append(s)
    else:
      j = self.rng.randrange(self.arrived[b][s.grade])
      if j < self.cap:
        cell[j] = s

  def pull(self, n: int = 1) -> int:
    """Read ``n`` more documents; the stream restarts when it ends (at most once per call without yielding anything)."""
    got, restarted = 0, False
    while got < n:
      try:
        self.add(next(self._it))
        got += 1
        restarted = False
      except StopIteration:
        if restarted:
          break
        self._it, restarted = iter(self._src), True
        self.passes += 1
    return got

  def _combos(self, b: int, gap: int) -> List[Tuple[int, int]]:
    have = [g for g in range(N_GRADES) if self.cells[b][g]]
    return [(hi, lo) for hi in have for lo in have if hi - lo >= gap]

  def _warm_up(self) -> None:
    budget = self.warm * N_GRADES * len(self.cells) * 64
    while budget > 0 and any(len(c) < self.warm for row in self.cells for c in row):
      if not self.pull(64):
        break
      budget -= 64

  # -- draws
  def draw(self, bucket: Optional[int] = None) -> Tuple[Labelled, Labelled]:
    if bucket is not None and self._barren.get(bucket) == sum(self.arrived[bucket]):
      return self.draw(None)        # nothing new arrived in this bucket since it last failed to make a pair
    buckets = [bucket] if bucket is not None else list(range(len(self.cells)))
    passes0, budget = self.passes, self.draw_budget

    def issue(cands, relaxed: bool):
      b, (hi, lo) = self.rng.choice(cands)
      self.issued += 1
      self.relaxed += int(relaxed)
      return self.rng.choice(self.cells[b][hi]), self.rng.choice(self.cells[b][lo])

    while True:
      strict = [(b, c) for b in buckets for c in self._combos(b, self.min_gap)]
      if strict:
        return issue(strict, False)
      loose = [(b, c) for b in buckets for c in self._combos(b, self.relaxed_gap)]
      under_cap = self.issued == 0 or self.relaxed + 1 <= self.max_relaxed_frac * (self.issued + 1)
      # past the cap, read on in the hope of a wider gap; a stream seen twice over has nothing new to offer
      exhausted = self.passes - passes0 >= 2 or budget <= 0
      if loose and (under_cap or exhausted):
        return issue(loose, True)
      if exhausted or not self.pull(64):
        break
      budget -= 64
    if bucket is not None:
      self._barren[bucket] = sum(self.arrived[bucket])
      return self.draw(None)        # this length bucket cannot make a pair: take one from any bucket
    raise RuntimeError("the graded stream never yields two documents of different grade and similar length")

  def next_pairs(self, n: int) -> List[Tuple[Labelled, Labelled]]:
    """``n`` pairs spread evenly over the length buckets, in random order."""
    if self.issued == 0:
      self._warm_up()
    nb = len(self.cells)
    out = [self.draw(i % nb) for i in range(n)]
    self.rng.shuffle(out)
    return out


# ---------------------------------------------------------------------------------------------- batches
def mix(sources: Sequence[Iterable[Labelled]], weights: Optional[Sequence[float]] = None, seed: int = 0) -> Iterator[Labelled]:
  """Endless weighted interleave; each source restarts when it runs out (a source that yields nothing is dropped)."""
  rng = random.Random(seed)
  srcs = list(sources)
  w = list(weights or [1.0] * len(srcs))
  its = [iter(s) for s in srcs]
  while srcs:
    k = rng.choices(range(len(srcs)), weights=w)[0]
    try:
      yield next(its[k])
    except StopIteration:
      its[k] = iter(srcs[k])
      try:
        yield next(its[k])
      except StopIteration:
        del srcs[k], w[k], its[k]


def probe_targets(samples: Sequence[Labelled], device="cpu") -> Dict[str, torch.Tensor]:
  """Targets for ``ProbeHead.loss``: NaN marks a missing regression target, -1 a missing class."""
  out: Dict[str, torch.Tensor] = {}
  for task, (_, kind) in PROBE_TASKS.items():
    if task == "domain":
      out[task] = torch.tensor([DOMAINS.get(s.domain, -1) for s in samples], dtype=torch.long, device=device)
    elif kind == "reg":
      out[task] = torch.tensor([s.signals.get(task, float("nan")) for s in samples], dtype=torch.float32, device=device)
    else:
      out[task] = torch.tensor([s.classes.get(task, -1) for s in samples], dtype=torch.long, device=device)
  return out


def probe_batches(stream: Iterable[Labelled], batch_size: int, encode: Callable[[str], List[int]], max_ctx: int,
                  device="cpu") -> Iterator[dict]:
  """Phase A batches ``{"docs", "targets"}``.  The gate has no weak label of its own; it learns in phase C."""
  buf: List[Labelled] = []
  for s in stream:
    buf.append(s)
    if len(buf) == batch_size:
      t = probe_targets(buf, device)
      t.pop("gate", None)
      yield {"docs": [x.ids(encode, max_ctx) for x in buf], "targets": t}
      buf = []


def judge_batches(oracle: Iterable[Labelled], batch_size: int, encode: Callable[[str], List[int]], max_ctx: int,
                  pairs: Optional[GradedPairs] = None, pairs_per_batch: int = 0, device="cpu") -> Iterator[dict]:
  """Phase B batches ``{"docs", "rubric", "pairs"}``: ``batch_size`` oracle-labelled documents, then ``pairs_per_batch``
  (better, worse) documents appended with an all-NaN rubric row and indexed by ``pairs`` [P, 2]."""
  nan = float("nan")
  for lab in _chunks(mix([oracle]), batch_size):
    docs = [x.ids(encode, max_ctx) for x in lab]
    rub = [list(x.rubric) if x.rubric is not None else [nan] * len(RUBRIC) for x in lab]
    idx: List[List[int]] = []
    if pairs is not None and pairs_per_batch > 0:
      for hi, lo in pairs.next_pairs(pairs_per_batch):
        idx.append([len(docs), len(docs) + 1])
        docs += [hi.ids(encode, max_ctx), lo.ids(encode, max_ctx)]
        rub += [[nan] * len(RUBRIC)] * 2
    yield {"docs": docs, "rubric": torch.tensor(rub, dtype=torch.float32, device=device),
           "pairs": torch.tensor(idx, dtype=torch.long, device=device).reshape(-1, 2)}


def _chunks(it: Iterable[Labelled], n: int) -> Iterator[List[Labelled]]:
  buf: List[Labelled] = []
  for x in it:
    buf.append(x)
    if len(buf) == n:
      yield buf
      buf = []
