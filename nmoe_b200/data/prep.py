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


# ------------------------------------------------------------------ Beam runner
# The same chain as a graph of three stages, so that a distributed runner can spread it over workers:
#   documents --tokenise (element-wise)--> (shard id, (doc id, tokens)) --group by shard--> write one shard family each
# With Apache Beam installed the stages become ParDo / GroupByKey / ParDo on any Beam runner (Dataflow, Flink, Direct);
# without it the built-in runner below executes the very same stage functions in this process, which is also how the
# stages are tested.  Documents inside a shard are written in doc-id order, so the output does not depend on the order
# in which a runner delivers a group.  Reference: nmoe/data/prep.py:404-537 (TokenizeDoFn, AssignShardDoFn, WriteShardDoFn).

def beam_tokenize_stage(cfg: PrepConfig):
  """element {"doc_id", "text"} -> zero or one (shard id, (doc id, token list))."""
  state = {}
  def fn(doc: dict):
    if "enc" not in state:                       # built on the worker, not pickled with the stage
      state["enc"] = get_tokenizer(cfg.tokenizer)
    text = normalize_text(doc["text"])
    if len(text) < cfg.min_chars:
      return
    toks = state["enc"].encode_ordinary(text)
    if toks:
      yield get_shard_id(doc["doc_id"], cfg.num_shards), (doc["doc_id"], toks)
  return fn


def beam_write_stage(cfg: PrepConfig, source_name: str):
  """(shard id, iterable of (doc id, tokens)) -> the manifest (as a dict) of that shard's files."""
  def fn(group):
    sid, docs = group
    vocab, eos = tokenizer_info(cfg.tokenizer)
    w = ShardedWriter(Path(cfg.output_dir), cfg.dataset, cfg.version, cfg.num_shards, cfg.tokenizer, vocab, eos,
                      shard_ids=[int(sid)], source_info={"source": source_name, **cfg.source_info})
    for _doc_id, toks in sorted(docs, key=lambda d: d[0]):
      w.add_document(int(sid), toks)
    yield w.finalize(write_manifest=False).to_dict()
  return fn


class LocalStageRunner:
  """In-process execution of the stage graph (flat-map, group-by-key, flat-map)."""

  def run(self, elements, tokenize, write) -> List[dict]:
    groups: Dict[int, list] = {}
    for el in elements:
      for k, v in tokenize(el):
        groups.setdefault(k, []).append(v)
    out: List[dict] = []
    for k in sorted(groups):
      out.extend(write((k, groups[k])))
    return out


def run_beam_pipeline(source: DataSource, cfg: PrepConfig, pipeline_options=None, runner: str = "auto") -> ManifestInfo:
  """Build the shards of ``source`` through the stage graph.  ``runner``: "beam" (needs apache_beam; ``pipeline_options``
  go to ``beam.Pipeline``), "local" (built-in), or "auto" (beam when importable)."""
  docs = ({"doc_id": d.doc_id, "text": d.text} for d in source)
  if cfg.max_documents:
    import itertools
    docs = itertools.islice(docs, cfg.max_documents)
  tokenize, write = beam_tokenize_stage(cfg), beam_write_stage(cfg, source.name)
  beam = None
  if runner in ("auto", "beam"):
    try:
      import apache_beam as beam  # type: ignore
    except ImportError:
      if runner == "beam":
        raise RuntimeError("runner='beam' needs the 'apache_beam' package (pip install apache-beam[gcp]); "
                           "runner='local' runs the same stages in this process")
  Path(cfg.output_dir).mkdir(parents=True, exist_ok=True)
  if beam is not None:
    parts_path = Path(cfg.output_dir) / "manifest.parts.jsonl"
    with beam.Pipeline(options=pipeline_options) as p:
      (p | "Documents" >> beam.Create(list(docs))
         | "Tokenize" >> beam.FlatMap(tokenize)
         | "ByShard" >> beam.GroupByKey()
         | "WriteShards" >> beam.FlatMap(write)
         | "ToJson" >> beam.Map(json.dumps)
         | "Parts" >> beam.io.WriteToText(str(parts_path), shard_name_template="", num_shards=1))
    parts = [json.loads(l) for l in parts_path.read_text().splitlines() if l.strip()]
    parts_path.unlink()
  else:
    parts = LocalStageRunner().run(docs, tokenize, write)
  if not parts:
    raise RuntimeError("the source produced no documents")
  m = merge_manifests([ManifestInfo.from_dict(p) for p in parts])
  write_manifest_file(Path(cfg.output_dir) / "manifest.json", m)
  return m


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
