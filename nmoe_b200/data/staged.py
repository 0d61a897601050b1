"""The data flow with every stage written to disk, so that an interrupted run picks up where it stopped.

``flow.run_flow`` streams documents through grading and rephrasing straight into the shard writers: nothing is kept in
between, which is right for a short job and wrong for one that spends GPU-days in the grading model.  This runner
executes the same specification as a chain of *stages*, each of which reads the previous stage's JSON-lines file and
appends to its own (nmoe/data/pipeline.py:22-466 keeps the same artefacts: raw documents, quality scores, kept
documents, rephrased documents, training shards):

    stages/raw.jsonl        documents as fetched from the source (this worker's slice)
    stages/scores.jsonl     one {"id", "score"} per graded document
    stages/kept.jsonl       documents whose score reaches the threshold, with the score in their metadata
    stages/rephrased.jsonl  rephrased versions (and the originals when asked for)
    <output_dir>/...        token shards, index files and manifest

A stage that finished is recorded in ``stages/state.json`` together with its row count and the digest of the
specification; a re-run skips it.  A stage that was interrupted is *continued*: ids already present in its output are
not computed again (a last line cut by the crash is dropped first).  A directory made under a different specification
is refused, as in ``run_flow``.
"""
from __future__ import annotations

import json
import os
from pathlib import Path
from typing import Callable, Dict, Iterable, Iterator, List, Optional

from .flow import FlowSpec, resolve_shard
from .prep import PrepConfig, PrepPipeline
from .sources import DataSource, Document, JSONLSource, create_source

STAGES = ("raw", "scores", "kept", "rephrased", "shards")


def _repair_tail(path: Path) -> None:
  """Drop a final line that does not end in a newline (the write a crash cut short)."""
  if not path.exists() or path.stat().st_size == 0:
    return
  with open(path, "rb+") as f:
    f.seek(-1, os.SEEK_END)
    if f.read(1) == b"\n":
      return
    data = path.read_bytes()
    f.truncate(data.rfind(b"\n") + 1)


def _rows(path: Path) -> Iterator[dict]:
  with open(path, encoding="utf-8") as f:
    for line in f:
      if line.strip():
        yield json.loads(line)


def _ids(path: Path, key: str = "id") -> set:
  return {str(r[key]) for r in _rows(path)} if path.exists() else set()


def _doc_row(d: Document) -> dict:
  return {"id": d.doc_id, "text": d.text, **{k: v for k, v in d.metadata.items() if k not in ("id", "text")}}


def _batched(it: Iterable, n: int) -> Iterator[list]:
  buf = []
  for x in it:
    buf.append(x)
    if len(buf) == n:
      yield buf
      buf = []
  if buf:
    yield buf


class StagedFlow:
  def __init__(self, spec: FlowSpec, *, grader: Optional[Callable[[List[str]], List[float]]] = None,
               rephraser: Optional[Callable[[List[str]], list]] = None, env: Optional[dict] = None,
               print_fn: Callable = print, source: Optional[DataSource] = None):
    self.spec, self.grader, self.rephraser, self.print = spec, grader, rephraser, print_fn
    self.idx, self.n = resolve_shard(spec, env)
    root = Path(spec.prep["output_dir"])
    self.out_dir = root if self.n == 1 else root / f"worker_{self.idx:04d}"
    self.dir = self.out_dir / "stages"
    self.dir.mkdir(parents=True, exist_ok=True)
    self._source = source
    self.state_path = self.dir / "state.json"
    self.state: Dict = json.loads(self.state_path.read_text()) if self.state_path.exists() else {"digest": spec.digest(), "done": {}}
    if self.state.get("digest") != spec.digest():
      raise RuntimeError(f"{self.out_dir} was produced by a different flow specification; use a new output_dir")
    self._save()

  # -- bookkeeping
  def _save(self) -> None:
    tmp = self.state_path.with_suffix(".tmp")
    tmp.write_text(json.dumps(self.state, indent=1))
    tmp.replace(self.state_path)

  def _finish(self, stage: str, rows: int) -> None:
    self.state["done"][stage] = rows
    self._save()
    self.print(f"[flow] worker {self.idx}/{self.n}: stage {stage} done ({rows:,} rows)")

  def done(self, stage: str) -> bool:
    return stage in self.state["done"]

  def path(self, stage: str) -> Path:
    return self.dir / f"{stage}.jsonl"

  # -- stages
  def fetch(self) -> Path:
    """Source -> raw.jsonl.  A source has no random access, so an interrupted fetch skips the ids it already wrote."""
    out = self.path("raw")
    if self.done("raw"):
      return out
    _repair_tail(out)
    have = _ids(out)
    src = self._source
    if src is None:
      kw = dict(self.spec.source)
      src = create_source(kw.pop("kind"), **kw)
    if self.n > 1:
      src = src.shard(self.idx, self.n)
    limit = self.spec.prep.get("max_documents")
    n = len(have)
    with open(out, "a", encoding="utf-8") as f:
      for d in src:
        if limit is not None and n >= int(limit):
          break
        if d.doc_id in have:
          continue
        f.write(json.dumps(_doc_row(d), ensure_ascii=False) + "\n")
        n += 1
    self._finish("raw", n)
    return out

  def grade(self, raw: Path) -> Path:
    """raw.jsonl -> scores.jsonl (every document) and kept.jsonl (score >= threshold)."""
    scores, kept = self.path("scores"), self.path("kept")
    if not self.spec.grade.get("enabled"):
      return raw
    thr = float(self.spec.grade.get("threshold", 0.5))
    if not self.done("scores"):
      if self.grader is None:
        raise RuntimeError("flow asks for grading but no grader was provided (load a HYDRA judge first)")
      _repair_tail(scores)
      have = _ids(scores)
      n = len(have)
      with open(scores, "a", encoding="utf-8") as f:
        todo = (r for r in _rows(raw) if str(r["id"]) not in have)
        for batch in _batched(todo, int(self.spec.grade.get("batch_size", 32))):
          for r, s in zip(batch, self.grader([r["text"] for r in batch])):
            f.write(json.dumps({"id": r["id"], "score": float(s)}) + "\n")
          f.flush()
          n += len(batch)
      self._finish("scores", n)
    if not self.done("kept"):
      # cheap and derived from two finished files: rebuilt from scratch rather than continued
      score = {str(r["id"]): r["score"] for r in _rows(scores)}
      n = 0
      with open(kept, "w", encoding="utf-8") as f:
        for r in _rows(raw):
          s = score.get(str(r["id"]))
          if s is not None and s >= thr:
            f.write(json.dumps({**r, "score": s}, ensure_ascii=False) + "\n")
            n += 1
      self._finish("kept", n)
    return kept

  def rephrase(self, prev: Path) -> Path:
    """kept.jsonl -> rephrased.jsonl: versions carry ``source_id`` so that a continued run knows what is finished."""
    rp = self.spec.rephrase
    if not rp.get("enabled"):
      return prev
    out = self.path("rephrased")
    if self.done("rephrased"):
      return out
    if self.rephraser is None:
      raise RuntimeError("flow asks for rephrasing but no rephraser was provided")
    _repair_tail(out)
    keep_original = bool(rp.get("keep_original", False))
    # a document is finished when its end marker was written: versions of a half-done document are written again
    # under the same ids, and the reader below keeps the last copy of an id
    finished = {str(r["source_id"]) for r in _rows(out) if r.get("end")} if out.exists() else set()
    n = 0
    with open(out, "a", encoding="utf-8") as f:
      todo = (r for r in _rows(prev) if str(r["id"]) not in finished)
      for batch in _batched(todo, int(rp.get("batch_size", 8))):
        for r, res in zip(batch, self.rephraser([r["text"] for r in batch])):
          versions = [res] if isinstance(res, str) else list(res)
          meta = {k: v for k, v in r.items() if k not in ("id", "text")}
          if keep_original:
            f.write(json.dumps({**r, "source_id": r["id"]}, ensure_ascii=False) + "\n")
          for v, t in enumerate(versions):
            if t:
              vid = r["id"] if len(versions) == 1 and not keep_original else f"{r['id']}#v{v}"
              f.write(json.dumps({**meta, "id": vid, "text": t, "source_id": r["id"], "rephrased": True, "version": v},
                                 ensure_ascii=False) + "\n")
          f.write(json.dumps({"source_id": r["id"], "end": True}) + "\n")
        f.flush()
    # compact: last copy of every id, end markers dropped
    last: Dict[str, dict] = {}
    for r in _rows(out):
      if not r.get("end"):
        last[str(r["id"])] = r
    tmp = out.with_suffix(".tmp")
    with open(tmp, "w", encoding="utf-8") as f:
      for r in last.values():
        f.write(json.dumps(r, ensure_ascii=False) + "\n")
        n += 1
    tmp.replace(out)
    self._finish("rephrased", n)
    return out

  def shards(self, prev: Path):
    if self.done("shards"):
      from .sinks import load_manifest
      return load_manifest(self.out_dir)
    p = dict(self.spec.prep)
    cfg = PrepConfig(output_dir=str(self.out_dir), dataset=p.get("dataset", "flow"), version=p.get("version", "v1"),
                     tokenizer=p.get("tokenizer", "o200k_harmony"), num_shards=int(p.get("num_shards", 8)),
                     max_tokens=p.get("max_tokens"), source_info={"flow_digest": self.spec.digest(), "staged": True})
    m = PrepPipeline(JSONLSource(str(prev)), cfg, print_fn=self.print).run()
    self._finish("shards", m.total_documents)
    return m

  def run(self):
    last = self.rephrase(self.grade(self.fetch()))
    m = self.shards(last)
    self.print(f"[flow] worker {self.idx}/{self.n}: {m.total_documents:,} documents, {m.total_tokens:,} tokens -> {self.out_dir}")
    return m


def run_flow_staged(spec: FlowSpec, **kw):
  return StagedFlow(spec, **kw).run()
