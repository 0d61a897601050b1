"""TOML-described data flow: raw documents -> (optional) quality grading -> keep -> (optional)
rephrase -> shard building (nmoe/data/flow.py:58-388).

Every section key can be overridden from the environment as ``NMOE_DATAFLOW__SECTION__KEY``.  Under a
Kubernetes Indexed job each pod takes the slice ``JOB_COMPLETION_INDEX`` of ``num_workers``.  A
``flow_spec.json`` written into the output directory guards against re-running a directory with a
different specification."""
from __future__ import annotations

import hashlib
import json
import os
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Callable, Dict, List, Optional

from ..config import load_toml
from .prep import PrepConfig, PrepPipeline
from .sources import DataSource, Document, FilteredSource, create_source


def apply_env_overrides(spec: Dict[str, Any], env: Optional[dict] = None) -> Dict[str, Any]:
  env = os.environ if env is None else env
  out = json.loads(json.dumps(spec))
  for k, v in env.items():
    if not k.startswith("NMOE_DATAFLOW__"):
      continue
    parts = k[len("NMOE_DATAFLOW__"):].lower().split("__")
    node = out
    for p in parts[:-1]:
      node = node.setdefault(p, {})
    try:
      node[parts[-1]] = json.loads(v)
    except json.JSONDecodeError:
      node[parts[-1]] = v
  return out


@dataclass
class FlowSpec:
  source: Dict[str, Any]
  prep: Dict[str, Any]
  grade: Dict[str, Any] = field(default_factory=dict)
  rephrase: Dict[str, Any] = field(default_factory=dict)
  shard: Dict[str, Any] = field(default_factory=dict)

  def digest(self) -> str:
    return hashlib.sha256(json.dumps(self.__dict__, sort_keys=True).encode()).hexdigest()


def resolve_shard(spec: FlowSpec, env: Optional[dict] = None):
  env = os.environ if env is None else env
  n = int(spec.shard.get("num_workers", env.get("NMOE_FLOW_WORKERS", 1)))
  i = int(spec.shard.get("index", env.get("JOB_COMPLETION_INDEX", 0)))
  if not 0 <= i < n:
    raise ValueError(f"worker index {i} outside [0, {n})")
  return i, n


def load_spec(path: Path, env: Optional[dict] = None) -> FlowSpec:
  d = apply_env_overrides(load_toml(path), env)
  return FlowSpec(source=d["source"], prep=d["prep"], grade=d.get("grade", {}), rephrase=d.get("rephrase", {}),
                  shard=d.get("shard", {}))


class _Mapped(DataSource):
  def __init__(self, base: DataSource, fn: Callable[[List[Document]], List[Document]], batch: int = 16):
    self.base, self.fn, self.batch = base, fn, batch
    self.name = f"mapped:{base.name}"

  def __iter__(self):
    buf: List[Document] = []
    for d in self.base:
      buf.append(d)
      if len(buf) == self.batch:
        yield from self.fn(buf)
        buf = []
    if buf:
      yield from self.fn(buf)


def run_flow(spec: FlowSpec, *, grader: Optional[Callable[[List[str]], List[float]]] = None,
             rephraser: Optional[Callable[[List[str]], List[str]]] = None, env: Optional[dict] = None,
             print_fn: Callable = print):
  """Runs the flow for this worker's slice and returns the shard manifest."""
  out_dir = Path(spec.prep["output_dir"])
  out_dir.mkdir(parents=True, exist_ok=True)
  guard = out_dir / "flow_spec.json"
  if guard.exists() and json.loads(guard.read_text()).get("digest") != spec.digest():
    raise RuntimeError(f"{out_dir} was produced by a different flow specification; use a new output_dir")
  guard.write_text(json.dumps({"digest": spec.digest(), "spec": spec.__dict__}, indent=1))
  src_kw = dict(spec.source)
  src: DataSource = create_source(src_kw.pop("kind"), **src_kw)
  idx, n = resolve_shard(spec, env)
  if n > 1:
    src = src.shard(idx, n)
  if spec.grade.get("enabled"):
    if grader is None:
      raise RuntimeError("flow asks for grading but no grader was provided (load a HYDRA judge first)")
    src = FilteredSource(src, float(spec.grade.get("threshold", 0.5)), score_fn=grader,
                         batch_size=int(spec.grade.get("batch_size", 32)))
  if spec.rephrase.get("enabled"):
    if rephraser is None:
      raise RuntimeError("flow asks for rephrasing but no rephraser was provided")
    keep_original = bool(spec.rephrase.get("keep_original", False))
    def _re(docs: List[Document]) -> List[Document]:
      # the rephraser answers one text per document, or a list of versions per document
      out: List[Document] = []
      for d, r in zip(docs, rephraser([d.text for d in docs])):
        if keep_original:
          out.append(d)
        versions = [r] if isinstance(r, str) else list(r)
        for v, t in enumerate(versions):
          if t:
            out.append(Document(d.doc_id if len(versions) == 1 else f"{d.doc_id}#v{v}", t,
                                {**d.metadata, "rephrased": True, "version": v}))
      return out
    src = _Mapped(src, _re, int(spec.rephrase.get("batch_size", 8)))
  p = dict(spec.prep)
  cfg = PrepConfig(output_dir=str(out_dir if n == 1 else out_dir / f"worker_{idx:04d}"), dataset=p.get("dataset", "flow"),
                   version=p.get("version", "v1"), tokenizer=p.get("tokenizer", "o200k_harmony"),
                   num_shards=int(p.get("num_shards", 8)), max_documents=p.get("max_documents"),
                   max_tokens=p.get("max_tokens"), source_info={"flow_digest": spec.digest()})
  m = PrepPipeline(src, cfg, print_fn=print_fn).run()
  print_fn(f"[flow] worker {idx}/{n}: {m.total_documents:,} documents, {m.total_tokens:,} tokens -> {cfg.output_dir}")
  return m
