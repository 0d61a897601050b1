"""Shard writers and manifests (nmoe/data/sinks.py:28-417).

A shard is a 1-D uint32 ``.npy`` of concatenated documents, each terminated by EOS, plus its
``.idx``.  Tokens stream to ``<name>.bin.tmp`` while a shard is open; ``finalize`` turns it into
the ``.npy`` (header + data, written next to it and renamed), writes the index and returns a
``ShardInfo`` with the file's sha256.  ``manifest.json`` lists every shard and is committed with
tmp + rename."""
from __future__ import annotations

import hashlib
import json
import struct
import time
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Any, Dict, List, Optional, Sequence

import numpy as np

from .errors import ManifestCommitError, ShardChecksumError, IndexMissingError
from .index import IndexWriter, index_path_for_shard
from .transforms import make_file_name


@dataclass
class ShardInfo:
  path: str
  index_path: str
  num_tokens: int
  num_documents: int
  checksum: str


@dataclass
class ManifestInfo:
  dataset: str
  version: str
  tokenizer: str
  vocab_size: int
  eos_token_id: int
  dtype: str
  created_at: str
  total_tokens: int
  total_documents: int
  num_shards: int
  shards: List[ShardInfo]
  source_info: Dict[str, Any] = field(default_factory=dict)

  def to_dict(self) -> Dict[str, Any]:
    return asdict(self)

  @classmethod
  def from_dict(cls, d: Dict[str, Any]) -> "ManifestInfo":
    d = dict(d)
    d["shards"] = [ShardInfo(**s) for s in d["shards"]]
    d.setdefault("source_info", {})
    return cls(**d)


def sha256_file(path: Path) -> str:
  h = hashlib.sha256()
  with open(path, "rb") as f:
    for chunk in iter(lambda: f.read(1 << 20), b""):
      h.update(chunk)
  return h.hexdigest()


class ShardWriter:
  """One shard: ``add_document`` appends tokens + EOS, ``finalize`` commits .npy + .idx."""

  def __init__(self, out_dir: Path, dataset: str, version: str, shard_idx: int, eos_token_id: int):
    self.out_dir = Path(out_dir)
    self.out_dir.mkdir(parents=True, exist_ok=True)
    self.path = self.out_dir / make_file_name(dataset, version, shard_idx)
    self.tmp = self.path.with_suffix(".bin.tmp")
    self.eos = eos_token_id
    self._f = open(self.tmp, "wb")
    self._n = 0
    self._idx = IndexWriter(index_path_for_shard(self.path))

  @property
  def num_tokens(self) -> int:
    return self._n

  def add_document(self, tokens: Sequence[int]) -> None:
    arr = np.empty(len(tokens) + 1, dtype="<u4")
    arr[:-1] = tokens
    arr[-1] = self.eos
    self._f.write(arr.tobytes())
    self._idx.add_document(self._n, self._n + len(arr))
    self._n += len(arr)

  def finalize(self) -> ShardInfo:
    self._f.close()
    data = np.memmap(self.tmp, dtype="<u4", mode="r", shape=(self._n,)) if self._n else np.empty(0, dtype="<u4")
    npy_tmp = self.path.with_suffix(".npy.tmp")
    with open(npy_tmp, "wb") as f:
      np.save(f, np.asarray(data))
    del data
    npy_tmp.replace(self.path)
    self.tmp.unlink(missing_ok=True)
    ndocs = self._idx.finalize()
    return ShardInfo(self.path.name, self._idx.path.name, self._n, ndocs, sha256_file(self.path))


class ShardedWriter:
  """Fan documents out over ``num_shards`` open shards (by a caller-supplied shard id)."""

  def __init__(self, out_dir: Path, dataset: str, version: str, num_shards: int, tokenizer: str, vocab_size: int,
               eos_token_id: int, shard_ids: Optional[Sequence[int]] = None, source_info: Optional[dict] = None):
    self.out_dir, self.dataset, self.version = Path(out_dir), dataset, version
    self.tokenizer, self.vocab_size, self.eos = tokenizer, vocab_size, eos_token_id
    self.source_info = source_info or {}
    ids = list(range(num_shards)) if shard_ids is None else list(shard_ids)
    self.writers = {i: ShardWriter(out_dir, dataset, version, i, eos_token_id) for i in ids}

  def add_document(self, shard_id: int, tokens: Sequence[int]) -> None:
    self.writers[shard_id].add_document(tokens)

  def finalize(self, write_manifest: bool = True) -> ManifestInfo:
    infos = [w.finalize() for _, w in sorted(self.writers.items())]
    m = ManifestInfo(self.dataset, self.version, self.tokenizer, self.vocab_size, self.eos, "uint32",
                     time.strftime("%Y-%m-%dT%H:%M:%SZ", time.gmtime()), sum(s.num_tokens for s in infos),
                     sum(s.num_documents for s in infos), len(infos), infos, self.source_info)
    if write_manifest:
      write_manifest_file(self.out_dir / "manifest.json", m)
    return m


def write_manifest_file(path: Path, m: ManifestInfo) -> None:
  tmp = Path(str(path) + ".tmp")
  try:
    tmp.write_text(json.dumps(m.to_dict(), indent=2))
    tmp.replace(path)
  except OSError as e:
    raise ManifestCommitError(f"could not commit {path}", str(e))


def load_manifest(path: Path) -> ManifestInfo:
  p = Path(path)
  if p.is_dir():
    p = p / "manifest.json"
  return ManifestInfo.from_dict(json.loads(p.read_text()))


def merge_manifests(parts: Sequence[ManifestInfo]) -> ManifestInfo:
  first = parts[0]
  shards = sorted((s for m in parts for s in m.shards), key=lambda s: s.path)
  return ManifestInfo(first.dataset, first.version, first.tokenizer, first.vocab_size, first.eos_token_id, first.dtype,
                      time.strftime("%Y-%m-%dT%H:%M:%SZ", time.gmtime()), sum(s.num_tokens for s in shards),
                      sum(s.num_documents for s in shards), len(shards), shards, first.source_info)


def verify_manifest(directory: Path, check_checksums: bool = True) -> ManifestInfo:
  """Every shard exists, its index is readable and tiles the shard, the token and document counts add up and
  (optionally) sha256 matches."""
  directory = Path(directory)
  m = load_manifest(directory)
  for s in m.shards:
    sp = directory / s.path
    if not (directory / s.index_path).exists():
      raise IndexMissingError(f"{s.index_path} is missing for shard {s.path}")
    if not sp.exists():
      raise ShardChecksumError(f"shard {s.path} is missing")
    n = int(np.load(sp, mmap_mode="r").shape[0])
    if n != s.num_tokens:
      raise ShardChecksumError(f"{s.path}: {n} tokens on disk, manifest says {s.num_tokens}")
    if check_checksums and sha256_file(sp) != s.checksum:
      raise ShardChecksumError(f"{s.path}: sha256 differs from the manifest")
    # the index must describe this shard: readable, as many documents as the manifest says, boundaries that tile
    # [0, num_tokens) in order.  A loader trusts these offsets without looking at the tokens.
    from .index import IndexReader
    try:
      b = IndexReader(directory / s.index_path).to_array()
    except (ValueError, OSError, struct.error) as e:
      raise IndexMissingError(f"{s.index_path} is unreadable: {e}; rebuild it with regenerate-index") from e
    if len(b) != s.num_documents:
      raise IndexMissingError(f"{s.index_path}: {len(b)} documents, manifest says {s.num_documents}")
    if len(b) and (int(b[0, 0]) != 0 or int(b[-1, 1]) != n or bool((b[1:, 0] != b[:-1, 1]).any()) or bool((b[:, 1] <= b[:, 0]).any())):
      raise IndexMissingError(f"{s.index_path}: document boundaries do not tile the shard's {n} tokens; rebuild it with regenerate-index")
  if sum(s.num_tokens for s in m.shards) != m.total_tokens:
    raise ShardChecksumError("manifest total_tokens does not match its shards")
  return m
