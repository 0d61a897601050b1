"""Shard building: stream documents -> normalise -> tokenise -> md5(doc_id) % num_shards -> shard writers
-> manifest (nmoe/data/prep.py:36-537).  ``ParallelPrepPipeline`` runs one process per worker, each
owning a disjoint set of output shards and scanning the whole source (documents of other shards
are skipped before tokenisation), then merges the per-worker manifests."""
from __future__ import annotations

import json
import multiprocessing as mp
import time
from dataclasses import dataclass, field
from pathlib import Path
from typing import Callable, Dict, List, Optional

from .errors import ResumeCursorMismatchError
from .sinks import ManifestInfo, ShardedWriter, load_manifest, merge_manifests, write_manifest_file
from .sources import DataSource
from .transforms import get_shard_id, get_tokenizer, normalize_text, tokenizer_info


@dataclass
class PrepConfig:
  output_dir: str
  dataset: str
  version: str = "v1"
  tokenizer: str = "o200k_harmony"
  num_shards: int = 8
  max_documents: Optional[int] = None
  max_tokens: Optional[int] = None
  min_chars: int = 1
  log_every: int = 10000
  source_info: Dict = field(default_factory=dict)


@dataclass
class PrepStats:
  documents: int = 0
  tokens: int = 0
  skipped: int = 0
  seconds: float = 0.0


class PrepPipeline:
  def __init__(self, source: DataSource, cfg: PrepConfig, shard_ids: Optional[List[int]] = None,
               print_fn: Callable = print):
    self.source, self.cfg, self.shard_ids, self.print = source, cfg, shard_ids, print_fn

  def run(self) -> ManifestInfo:
    cfg = self.cfg
    vocab, eos = tokenizer_info(cfg.tokenizer)
    enc = get_tokenizer(cfg.tokenizer)
    mine = set(self.shard_ids) if self.shard_ids is not None else None
    writer = ShardedWriter(Path(cfg.output_dir), cfg.dataset, cfg.version, cfg.num_shards, cfg.tokenizer, vocab, eos,
                           shard_ids=self.shard_ids, source_info={"source": self.source.name, **cfg.source_info})
    st = PrepStats()
    t0 = time.time()
    for doc in self.source:
      sid = get_shard_id(doc.doc_id, cfg.num_shards)
      if mine is not None and sid not in mine:
        continue
      text = normalize_text(doc.text)
      if len(text) < cfg.min_chars:
        st.skipped += 1
        continue
      toks = enc.encode_ordinary(text)
      if not toks:
        st.skipped += 1
        continue
      writer.add_document(sid, toks)
      st.documents += 1
      st.tokens += len(toks) + 1
      if cfg.log_every and st.documents % cfg.log_every == 0:
        self.print(f"[prep] {st.documents:,} docs {st.tokens:,} tokens {st.tokens / max(1e-9, time.time() - t0):,.0f} tok/s")
      if (cfg.max_documents and st.documents >= cfg.max_documents) or (cfg.max_tokens and st.tokens >= cfg.max_tokens):
        break
    st.seconds = time.time() - t0
    part = self.shard_ids is not None
    m = writer.finalize(write_manifest=not part)
    if part:
      write_manifest_file(Path(cfg.output_dir) / f"manifest.part{min(self.shard_ids):06d}.json", m)
    self.stats = st
    return m


def _worker(args):
  source_factory, cfg, shard_ids = args
  return PrepPipeline(source_factory(), cfg, shard_ids, print_fn=lambda *a: None).run().to_dict()


class ParallelPrepPipeline:
  def __init__(self, source_factory: Callable[[], DataSource], cfg: PrepConfig, workers: int = 4):
    self.source_factory, self.cfg, self.workers = source_factory, cfg, max(1, workers)

  def run(self) -> ManifestInfo:
    groups = [list(range(w, self.cfg.num_shards, self.workers)) for w in range(self.workers)]
    groups = [g for g in groups if g]
    # forked workers inherit the factory (no pickling); each leaves a manifest.partNNNNNN.json behind
    ctx = mp.get_context("fork")
    procs = [ctx.Process(target=_worker, args=((self.source_factory, self.cfg, g),)) for g in groups]
    for p in procs:
      p.start()
    for p in procs:
      p.join()
    bad = [p.exitcode for p in procs if p.exitcode != 0]
    if bad:
      raise RuntimeError(f"{len(bad)} prep worker(s) failed (exit codes {bad})")
    parts = [load_manifest(Path(self.cfg.output_dir) / f"manifest.part{min(g):06d}.json").to_dict() for g in groups]
    m = merge_manifests([ManifestInfo.from_dict(p) for p in parts])
    write_manifest_file(Path(self.cfg.output_dir) / "manifest.json", m)
    for p in Path(self.cfg.output_dir).glob("manifest.part*.json"):
      p.unlink()
    return m


def run_beam_pipeline(*_a, **_k):
  """Apache Beam runner of the same transform chain; Beam is an optional dependency."""
  try:
    import apache_beam  # noqa: F401
  except ImportError as e:
    raise RuntimeError("the Beam runner needs the 'apache_beam' package; use ParallelPrepPipeline instead") from e
  raise NotImplementedError("Beam runner: wire PrepPipeline's transforms into a beam.Pipeline for your runner")


class ResumeState:
  """``state.json`` next to the output: last processed doc id + its checksum, to detect a changed source."""

  def __init__(self, path: Path):
    self.path = Path(path)

  def save(self, doc_id: str, checksum: str, n_docs: int) -> None:
    self.path.write_text(json.dumps({"doc_id": doc_id, "checksum": checksum, "documents": n_docs}))

  def check(self, doc_id: str, checksum: str) -> None:
    if not self.path.exists():
      return
    st = json.loads(self.path.read_text())
    if st["doc_id"] == doc_id and st["checksum"] != checksum:
      raise ResumeCursorMismatchError(f"document {doc_id} changed since the last run")
