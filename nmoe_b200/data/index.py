"""Document-boundary index next to each shard (nmoe/data/index.py:32-161).

``.idx`` = 32-byte header (magic ``NMOEIDX\\0``, version u64 = 1, num_docs u64, reserved u64) followed
by ``num_docs`` little-endian (start, end) u64 pairs; start inclusive, end exclusive, EOS included."""
from __future__ import annotations

import struct
from pathlib import Path
from typing import Iterator, List, Tuple

import numpy as np

INDEX_MAGIC = b"NMOEIDX\x00"
INDEX_VERSION = 1
HEADER_SIZE = 32


def pack_header(num_docs: int) -> bytes:
  return struct.pack("<8sQQQ", INDEX_MAGIC, INDEX_VERSION, num_docs, 0)


def unpack_header(data: bytes) -> int:
  magic, version, num_docs, _ = struct.unpack("<8sQQQ", data[:HEADER_SIZE])
  if magic != INDEX_MAGIC:
    raise ValueError(f"bad index magic {magic!r}")
  if version != INDEX_VERSION:
    raise ValueError(f"unsupported index version {version}")
  return int(num_docs)


class IndexWriter:
  def __init__(self, path: Path):
    self.path = Path(path)
    self._b: List[Tuple[int, int]] = []

  def add_document(self, start: int, end: int) -> None:
    self._b.append((start, end))

  def finalize(self) -> int:
    tmp = self.path.with_suffix(".idx.tmp")
    with open(tmp, "wb") as f:
      f.write(pack_header(len(self._b)))
      f.write(np.asarray(self._b, dtype="<u8").reshape(-1).tobytes())
    tmp.replace(self.path)
    return len(self._b)


class IndexReader:
  def __init__(self, path: Path):
    self.path = Path(path)
    with open(self.path, "rb") as f:
      self.num_docs = unpack_header(f.read(HEADER_SIZE))
      self._b = np.frombuffer(f.read(), dtype="<u8").reshape(-1, 2)
    if len(self._b) != self.num_docs:
      raise ValueError(f"{path}: header says {self.num_docs} documents, body has {len(self._b)}")

  def get_document(self, i: int) -> Tuple[int, int]:
    if not 0 <= i < self.num_docs:
      raise IndexError(f"document {i} out of range [0, {self.num_docs})")
    return int(self._b[i, 0]), int(self._b[i, 1])

  def iter_documents(self) -> Iterator[Tuple[int, int]]:
    for s, e in self._b:
      yield int(s), int(e)

  def to_array(self) -> np.ndarray:
    return self._b.copy()


def index_path_for_shard(shard: Path) -> Path:
  return Path(shard).with_suffix(".idx")


def regenerate_index_from_shard(shard: Path, eos_token_id: int) -> Path:
  """Rebuild the .idx by scanning the shard for EOS tokens (a trailing unterminated run counts as a document)."""
  tokens = np.load(shard, mmap_mode="r")
  eos = np.flatnonzero(np.asarray(tokens) == eos_token_id)
  w = IndexWriter(index_path_for_shard(shard))
  start = 0
  for p in eos:
    w.add_document(start, int(p) + 1)
    start = int(p) + 1
  if start < len(tokens):
    w.add_document(start, len(tokens))
  w.finalize()
  return w.path
