"""Document sources (nmoe/data/sources.py:60-878): an iterator of ``Document(doc_id, text, metadata)``
with deterministic ids, shardable across workers.  Local formats (JSONL, JSONL.zst, plain text,
Arrow/Parquet) are always available; HuggingFace sources need the ``datasets`` /
``huggingface_hub`` packages and network access and raise a SourceNotFoundError otherwise."""
from __future__ import annotations

import glob
import hashlib
import io
import json
import os
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Callable, Dict, Iterator, List, Optional

from .errors import SourceNotFoundError


@dataclass
class Document:
  doc_id: str
  text: str
  metadata: Dict[str, Any] = field(default_factory=dict)


class DataSource:
  name = "source"

  def __iter__(self) -> Iterator[Document]:
    raise NotImplementedError

  def shard(self, index: int, count: int) -> "DataSource":
    """A view that yields every ``count``-th document starting at ``index`` (stable order)."""
    return _StridedSource(self, index, count)

  def estimate_size(self) -> Optional[int]:
    return None


class _StridedSource(DataSource):
  def __init__(self, base: DataSource, index: int, count: int):
    self.base, self.index, self.count = base, index, count
    self.name = f"{base.name}[{index}/{count}]"

  def __iter__(self):
    for i, d in enumerate(self.base):
      if i % self.count == self.index:
        yield d


def _expand(paths) -> List[str]:
  if isinstance(paths, (str, Path)):
    paths = [paths]
  out: List[str] = []
  for p in paths:
    p = str(p)
    if os.path.isdir(p):
      out += sorted(glob.glob(os.path.join(p, "**", "*"), recursive=True))
    else:
      out += sorted(glob.glob(p, recursive=True)) or ([p] if os.path.exists(p) else [])
  return [p for p in out if os.path.isfile(p)]


def _doc_id(prefix: str, i: int, obj: Optional[dict], id_field: Optional[str]) -> str:
  if obj is not None and id_field and id_field in obj:
    return str(obj[id_field])
  return f"{prefix}:{i}"


class JSONLSource(DataSource):
  def __init__(self, paths, text_field: str = "text", id_field: Optional[str] = "id"):
    self.files = [p for p in _expand(paths) if p.endswith((".jsonl", ".json", ".ndjson"))]
    if not self.files:
      raise SourceNotFoundError(f"no .jsonl files under {paths}")
    self.text_field, self.id_field = text_field, id_field
    self.name = f"jsonl:{Path(self.files[0]).parent.name}"

  def _lines(self, path: str) -> Iterator[str]:
    with open(path, "r", encoding="utf-8") as f:
      yield from f

  def __iter__(self):
    for path in self.files:
      stem = Path(path).name
      for i, line in enumerate(self._lines(path)):
        line = line.strip()
        if not line:
          continue
        try:
          obj = json.loads(line)
        except json.JSONDecodeError:
          continue
        text = obj.get(self.text_field)
        if isinstance(text, str) and text:
          meta = {k: v for k, v in obj.items() if k != self.text_field}
          yield Document(_doc_id(stem, i, obj, self.id_field), text, meta)


class JSONLZstSource(JSONLSource):
  """``.jsonl.zst`` files; needs the ``zstandard`` package."""

  def __init__(self, paths, text_field: str = "text", id_field: Optional[str] = "id"):
    self.files = [p for p in _expand(paths) if p.endswith(".zst")]
    if not self.files:
      raise SourceNotFoundError(f"no .zst files under {paths}")
    self.text_field, self.id_field = text_field, id_field
    self.name = f"jsonl.zst:{Path(self.files[0]).parent.name}"

  def _lines(self, path: str) -> Iterator[str]:
    try:
      import zstandard
    except ImportError as e:
      raise SourceNotFoundError("reading .zst needs the 'zstandard' package", str(e))
    with open(path, "rb") as f:
      reader = zstandard.ZstdDecompressor().stream_reader(f)
      yield from io.TextIOWrapper(reader, encoding="utf-8")


class TextFileSource(DataSource):
  """One document per file, or per paragraph block with ``split_on`` (e.g. a blank line)."""

  def __init__(self, paths, split_on: Optional[str] = None, suffixes=(".txt", ".md")):
    self.files = [p for p in _expand(paths) if p.endswith(tuple(suffixes))]
    if not self.files:
      raise SourceNotFoundError(f"no text files under {paths}")
    self.split_on = split_on
    self.name = f"text:{Path(self.files[0]).parent.name}"

  def __iter__(self):
    for path in self.files:
      text = Path(path).read_text(encoding="utf-8", errors="replace")
      if self.split_on is None:
        yield Document(Path(path).name, text, {"path": path})
      else:
        for i, part in enumerate(text.split(self.split_on)):
          if part.strip():
            yield Document(f"{Path(path).name}:{i}", part, {"path": path})


class ArrowSource(DataSource):
  """Arrow IPC / Parquet files through pyarrow, read batch by batch."""

  def __init__(self, paths, text_field: str = "text", id_field: Optional[str] = "id"):
    self.files = [p for p in _expand(paths) if p.endswith((".arrow", ".parquet", ".feather"))]
    if not self.files:
      raise SourceNotFoundError(f"no arrow/parquet files under {paths}")
    self.text_field, self.id_field = text_field, id_field
    self.name = f"arrow:{Path(self.files[0]).parent.name}"

  def __iter__(self):
    import pyarrow as pa
    import pyarrow.parquet as pq
    for path in self.files:
      if path.endswith(".parquet"):
        batches = pq.ParquetFile(path).iter_batches(batch_size=1024)
      else:
        try:
          batches = pa.ipc.open_file(path).read_all().to_batches(1024)
        except pa.ArrowInvalid:
          batches = pa.ipc.open_stream(path).read_all().to_batches(1024)
      n = 0
      for b in batches:
        cols = b.to_pydict()
        texts = cols.get(self.text_field, [])
        ids = cols.get(self.id_field) if self.id_field else None
        for j, t in enumerate(texts):
          if isinstance(t, str) and t:
            yield Document(str(ids[j]) if ids else f"{Path(path).name}:{n}", t, {})
          n += 1


class HuggingFaceSource(DataSource):
  """Streaming ``datasets.load_dataset``; ``shard`` maps to the dataset's own sharding."""

  def __init__(self, dataset: str, subset: Optional[str] = None, split: str = "train", text_field: str = "text",
               data_files=None, id_field: Optional[str] = "id"):
    self.dataset, self.subset, self.split = dataset, subset, split
    self.text_field, self.data_files, self.id_field = text_field, data_files, id_field
    self.name = f"hf:{dataset}"
    self._shard = None

  def shard(self, index: int, count: int) -> "HuggingFaceSource":
    s = HuggingFaceSource(self.dataset, self.subset, self.split, self.text_field, self.data_files, self.id_field)
    s._shard = (index, count)
    return s

  def __iter__(self):
    try:
      import datasets
      ds = datasets.load_dataset(self.dataset, self.subset, split=self.split, streaming=True,
                                 data_files=self.data_files)
    except Exception as e:
      raise SourceNotFoundError(f"cannot open HuggingFace dataset {self.dataset}", str(e))
    if self._shard is not None:
      i, n = self._shard
      ds = ds.shard(num_shards=n, index=i) if getattr(ds, "n_shards", 1) >= n else ds
    for k, row in enumerate(ds):
      if self._shard is not None and getattr(ds, "n_shards", 1) < self._shard[1] and k % self._shard[1] != self._shard[0]:
        continue
      t = row.get(self.text_field)
      if isinstance(t, str) and t:
        yield Document(_doc_id(self.dataset, k, row, self.id_field), t, {})


class HfFileSystemSource(DataSource):
  """Raw files of a dataset repository through ``huggingface_hub.HfFileSystem`` (jsonl / jsonl.zst)."""

  def __init__(self, repo: str, pattern: str, text_field: str = "text"):
    self.repo, self.pattern, self.text_field = repo, pattern, text_field
    self.name = f"hffs:{repo}"

  def __iter__(self):
    try:
      from huggingface_hub import HfFileSystem
      fs = HfFileSystem()
      files = sorted(fs.glob(f"datasets/{self.repo}/{self.pattern}"))
    except Exception as e:
      raise SourceNotFoundError(f"cannot list {self.repo}/{self.pattern}", str(e))
    for path in files:
      with fs.open(path, "rb") as f:
        stream = f
        if path.endswith(".zst"):
          import zstandard
          stream = zstandard.ZstdDecompressor().stream_reader(f)
        for i, line in enumerate(io.TextIOWrapper(stream, encoding="utf-8")):
          try:
            obj = json.loads(line)
          except json.JSONDecodeError:
            continue
          t = obj.get(self.text_field)
          if isinstance(t, str) and t:
            yield Document(f"{Path(path).name}:{i}", t, {})


class ScoringSource(DataSource):
  """Wraps a source and attaches ``metadata['score']`` from a grading function (HYDRA scoring wrapper)."""

  def __init__(self, base: DataSource, score_fn: Callable[[List[str]], List[float]], batch_size: int = 32):
    self.base, self.score_fn, self.batch_size = base, score_fn, batch_size
    self.name = f"scored:{base.name}"

  def __iter__(self):
    buf: List[Document] = []
    for d in self.base:
      buf.append(d)
      if len(buf) == self.batch_size:
        yield from self._flush(buf)
        buf = []
    if buf:
      yield from self._flush(buf)

  def _flush(self, docs):
    for d, s in zip(docs, self.score_fn([d.text for d in docs])):
      d.metadata["score"] = float(s)
      yield d


class FilteredSource(DataSource):
  """Keeps documents whose score (computed by ``score_fn`` or already in metadata) is >= ``threshold``."""

  def __init__(self, base: DataSource, threshold: float, score_fn: Optional[Callable] = None, batch_size: int = 32):
    self.base = ScoringSource(base, score_fn, batch_size) if score_fn is not None else base
    self.threshold = threshold
    self.name = f"filtered:{base.name}"
    self.seen = self.kept = 0

  def __iter__(self):
    for d in self.base:
      self.seen += 1
      if float(d.metadata.get("score", float("-inf"))) >= self.threshold:
        self.kept += 1
        yield d


class AuditedSource(DataSource):
  """Passes a scored source through and writes one ``{"id", "score", "kept"}`` line per document seen, kept or not, to
  ``{audit_dir}/scores.jsonl``: the trail that shows what a quality filter dropped (``prep --hydra-audit-dir``).
  With ``threshold=None`` nothing is dropped and ``kept`` is always true."""

  def __init__(self, base: DataSource, audit_dir, threshold: Optional[float] = None, snippet_chars: int = 160):
    self.base, self.dir, self.threshold, self.snippet = base, Path(audit_dir), threshold, snippet_chars
    self.name = f"audited:{base.name}"
    self.seen = self.kept = 0

  def __iter__(self):
    self.dir.mkdir(parents=True, exist_ok=True)
    with open(self.dir / "scores.jsonl", "a", encoding="utf-8") as f:
      for d in self.base:
        score = float(d.metadata.get("score", float("nan")))
        keep = self.threshold is None or score >= self.threshold
        self.seen += 1
        self.kept += int(keep)
        f.write(json.dumps({"id": d.doc_id, "score": score, "kept": keep, "snippet": d.text[:self.snippet]}, ensure_ascii=False) + "\n")
        if keep:
          yield d
    (self.dir / "summary.json").write_text(json.dumps({"seen": self.seen, "kept": self.kept, "threshold": self.threshold}))


def content_doc_id(text: str) -> str:
  return hashlib.sha1(text.encode("utf-8")).hexdigest()[:20]


def create_source(kind: str, **kw) -> DataSource:
  kinds = {"jsonl": JSONLSource, "jsonl_zst": JSONLZstSource, "text": TextFileSource, "arrow": ArrowSource,
           "parquet": ArrowSource, "hf": HuggingFaceSource, "huggingface": HuggingFaceSource,
           "hffs": HfFileSystemSource}
  if kind in ("arxiv_tars", "ar5iv", "arxiv_paired"):
    from . import arxiv_sources as A      # imports this module, hence not at the top
    return {"arxiv_tars": A.ArxivTarSource, "ar5iv": A.Ar5ivSource, "arxiv_paired": A.ArxivPairedSource}[kind](**kw)
  if kind not in kinds:
    raise SourceNotFoundError(f"unknown source kind '{kind}'; expected one of {sorted(kinds) + ['ar5iv', 'arxiv_paired', 'arxiv_tars']}")
  return kinds[kind](**kw)
