"""Exact and near-duplicate removal (nmoe/data/dedup.py:34-227): sha1 over normalised text for exact
duplicates; MinHash signatures over word shingles with banded LSH for near duplicates, streamed;
repeated lines / paragraphs inside one document (nmoe/data/dedup.py:47-68)."""
from __future__ import annotations

import hashlib
import re
from collections import defaultdict
from typing import Dict, Iterable, Iterator, List, Set, Tuple

import numpy as np

from .sources import Document
from .transforms import normalize_text

_MERSENNE = (1 << 61) - 1
_WORD = re.compile(r"\w+", re.UNICODE)


def dedup_exact(docs: Iterable[Document]) -> Iterator[Document]:
  seen: Set[bytes] = set()
  for d in docs:
    h = hashlib.sha1(normalize_text(d.text).lower().encode("utf-8")).digest()
    if h not in seen:
      seen.add(h)
      yield d


def _key(s: str) -> str:
  return " ".join(s.split()).lower()


def dedup_within(text: str, unit: str = "lines", min_chars: int = 12) -> str:
  """Drop later repeats of a line (``unit="lines"``) or of a blank-line-separated paragraph (``"paragraphs"``) inside
  one document: navigation bars, cookie banners and footers that a page repeats.  Units are compared after collapsing
  white space and case; units shorter than ``min_chars`` (list bullets, braces, "}" lines of code) are never dropped,
  and neither are blank lines, so the document keeps its shape."""
  if unit not in ("lines", "paragraphs"):
    raise ValueError("unit must be 'lines' or 'paragraphs'")
  sep = "\n" if unit == "lines" else "\n\n"
  parts = text.split(sep) if unit == "lines" else re.split(r"\n\s*\n", text)
  seen: Set[str] = set()
  out: List[str] = []
  for p in parts:
    k = _key(p)
    if len(k) >= min_chars:
      if k in seen:
        continue
      seen.add(k)
    out.append(p)
  return sep.join(out)


def dedup_within_docs(docs: Iterable[Document], unit: str = "lines", min_chars: int = 12) -> Iterator[Document]:
  for d in docs:
    t = dedup_within(d.text, unit, min_chars)
    if t.strip():
      yield Document(d.doc_id, t, d.metadata) if t != d.text else d


def shingles(text: str, k: int = 5) -> Set[int]:
  words = _WORD.findall(text.lower())
  if len(words) < k:
    words = words + [""] * (k - len(words))
  return {int.from_bytes(hashlib.blake2b(" ".join(words[i:i + k]).encode(), digest_size=8).digest(), "little")
          for i in range(len(words) - k + 1)}


class MinHasher:
  def __init__(self, num_perm: int = 128, seed: int = 1):
    rng = np.random.default_rng(seed)
    self.a = rng.integers(1, _MERSENNE, size=num_perm, dtype=np.uint64)
    self.b = rng.integers(0, _MERSENNE, size=num_perm, dtype=np.uint64)
    self.num_perm = num_perm

  def signature(self, text: str, k: int = 5) -> np.ndarray:
    sh = np.fromiter(shingles(text, k), dtype=np.uint64)
    if sh.size == 0:
      return np.full(self.num_perm, np.iinfo(np.uint64).max, dtype=np.uint64)
    # (a * x + b) mod p with python-int safety via object arithmetic on small chunks
    x = sh.astype(object)
    sig = np.empty(self.num_perm, dtype=np.uint64)
    for i in range(self.num_perm):
      sig[i] = min((int(self.a[i]) * int(v) + int(self.b[i])) % _MERSENNE for v in x)
    return sig


def minhash_signature(text: str, num_perm: int = 128, k: int = 5, seed: int = 1) -> np.ndarray:
  return MinHasher(num_perm, seed).signature(text, k)


def jaccard_estimate(a: np.ndarray, b: np.ndarray) -> float:
  return float((a == b).mean())


class LSHIndex:
  """Banded LSH: two signatures collide if any band of ``rows`` values is identical."""

  def __init__(self, num_perm: int = 128, bands: int = 32):
    assert num_perm % bands == 0
    self.bands, self.rows = bands, num_perm // bands
    self.tables: List[Dict[bytes, List[int]]] = [defaultdict(list) for _ in range(bands)]
    self.sigs: List[np.ndarray] = []

  def query(self, sig: np.ndarray) -> Set[int]:
    out: Set[int] = set()
    for b in range(self.bands):
      out.update(self.tables[b].get(sig[b * self.rows:(b + 1) * self.rows].tobytes(), ()))
    return out

  def insert(self, sig: np.ndarray) -> int:
    i = len(self.sigs)
    self.sigs.append(sig)
    for b in range(self.bands):
      self.tables[b][sig[b * self.rows:(b + 1) * self.rows].tobytes()].append(i)
    return i


def stream_near_dedup(docs: Iterable[Document], threshold: float = 0.8, num_perm: int = 64, bands: int = 16,
                      k: int = 5) -> Iterator[Document]:
  """Yields documents whose estimated Jaccard similarity to every earlier kept document is < threshold."""
  mh = MinHasher(num_perm)
  idx = LSHIndex(num_perm, bands)
  for d in docs:
    sig = mh.signature(d.text, k)
    if any(jaccard_estimate(sig, idx.sigs[c]) >= threshold for c in idx.query(sig)):
      continue
    idx.insert(sig)
    yield d
