"""Shard-native document references: a document named by where its tokens already sit.

Once a corpus is tokenised into ``.npy`` shards, later stages (grading, oracle labelling, head training) should not
carry the text around again.  A reference is the string

    {source}//{shard path relative to the data root}#s={start}:e={end}

with ``start`` inclusive and ``end`` exclusive token offsets into the shard (the same pairs the shard's ``.idx`` file
holds).  The string form is a data contract with other tools that read and write these ids
(nmoe/data/docid.py:1-54), so it is kept byte for byte; everything around it here is this package's own:
``SpanRef`` parses and prints it, ``SpanReader`` serves tokens for many references with one memory map per shard,
``enumerate_refs`` lists every document of a prepared dataset, and ``sample_refs`` draws a reproducible subset.
"""
from __future__ import annotations

import hashlib
import re
from collections import OrderedDict
from dataclasses import dataclass
from pathlib import Path
from typing import Iterable, Iterator, List, Optional, Sequence

import numpy as np

from .index import IndexReader, index_path_for_shard

_REF = re.compile(r"^(?P<source>.*?)//(?P<rel>[^#]+)#s=(?P<s>\d+):e=(?P<e>\d+)$")


@dataclass(frozen=True)
class SpanRef:
  source: str
  rel_path: str
  start: int
  end: int

  def __post_init__(self):
    if self.start < 0 or self.end < self.start:
      raise ValueError(f"bad token span [{self.start}, {self.end})")
    if "//" in self.source or "#" in self.rel_path:
      raise ValueError("source must not contain '//' and the shard path must not contain '#'")

  def __str__(self) -> str:
    return f"{self.source}//{self.rel_path}#s={self.start}:e={self.end}"

  def __len__(self) -> int:
    return self.end - self.start

  @classmethod
  def parse(cls, text: str) -> "SpanRef":
    m = _REF.match(text.strip())
    if m is None:
      raise ValueError(f"not a shard reference (want source//path.npy#s=START:e=END): {text!r}")
    return cls(m["source"], m["rel"], int(m["s"]), int(m["e"]))

  @classmethod
  def make(cls, source: str, rel_path, start: int, end: int) -> "SpanRef":
    """Normalises the path the way the string form wants it: forward slashes, no leading slash."""
    return cls(source, str(rel_path).replace("\\", "/").lstrip("/"), int(start), int(end))

  def path(self, data_root) -> Path:
    p = (Path(data_root) / self.rel_path).resolve()
    root = Path(data_root).resolve()
    if root != p and root not in p.parents:      # "../" in a reference must not leave the data root
      raise ValueError(f"{self.rel_path!r} points outside {data_root}")
    return p


def is_ref(text: str) -> bool:
  return _REF.match(text.strip()) is not None


class SpanReader:
  """Tokens for references under one data root.  Shards are memory-mapped on first use and the ``max_open`` most
  recently used maps are kept, so reading a shuffled list of references does not reopen a file per document."""

  def __init__(self, data_root, max_open: int = 64):
    self.root, self.max_open = Path(data_root), max_open
    self._maps: "OrderedDict[str, np.ndarray]" = OrderedDict()

  def _shard(self, ref: SpanRef) -> np.ndarray:
    m = self._maps.get(ref.rel_path)
    if m is None:
      m = np.load(ref.path(self.root), mmap_mode="r")
      self._maps[ref.rel_path] = m
      while len(self._maps) > self.max_open:
        self._maps.popitem(last=False)
    else:
      self._maps.move_to_end(ref.rel_path)
    return m

  def tokens(self, ref, max_tokens: Optional[int] = None, drop_eos: Optional[int] = None) -> List[int]:
    ref = SpanRef.parse(ref) if isinstance(ref, str) else ref
    shard = self._shard(ref)
    if ref.end > shard.shape[0]:
      raise ValueError(f"{ref}: the shard holds {shard.shape[0]} tokens")
    ids = np.asarray(shard[ref.start:ref.end]).astype(np.int64)
    if drop_eos is not None and len(ids) and ids[-1] == drop_eos:
      ids = ids[:-1]
    return ids[:max_tokens].tolist() if max_tokens is not None else ids.tolist()


def enumerate_refs(data_root, source: str, subdir: str = "", min_tokens: int = 0) -> Iterator[SpanRef]:
  """Every document of every shard under ``data_root/subdir`` that has an index file, in path then offset order."""
  root = Path(data_root)
  for shard in sorted((root / subdir).rglob("*.npy")):
    idx = index_path_for_shard(shard)
    if not idx.is_file():
      continue
    rel = shard.relative_to(root).as_posix()
    for s, e in IndexReader(idx).iter_documents():
      if e - s >= min_tokens:
        yield SpanRef(source, rel, int(s), int(e))


def sample_refs(refs: Iterable[SpanRef], fraction: float, seed: int = 0) -> Iterator[SpanRef]:
  """A subset chosen by a hash of (seed, reference): the same references come back however the input is ordered or
  split among workers, and growing ``fraction`` only adds documents."""
  if not 0.0 <= fraction <= 1.0:
    raise ValueError("fraction must lie in [0, 1]")
  cut = int(fraction * (1 << 64))
  for r in refs:
    h = int.from_bytes(hashlib.blake2b(f"{seed}:{r}".encode(), digest_size=8).digest(), "big")
    if h < cut:
      yield r


def write_refs(path, refs: Iterable[SpanRef]) -> int:
  """One ``{"doc_id": ...}`` JSON object per line: the list format the grading commands read."""
  import json
  n = 0
  with open(path, "w", encoding="utf-8") as f:
    for r in refs:
      f.write(json.dumps({"doc_id": str(r), "source": r.source, "tokens": len(r)}) + "\n")
      n += 1
  return n


def read_refs(path, skip: Sequence[str] = ()) -> Iterator[SpanRef]:
  import json
  seen = set(skip)
  with open(path, encoding="utf-8") as f:
    for line in f:
      line = line.strip()
      if not line:
        continue
      did = json.loads(line).get("doc_id")
      if did and did not in seen:
        yield SpanRef.parse(did)
