"""The task registry: which corpora exist, where their shards are, what they are built from, and how.

``configs/tasks.toml`` holds a ``[corpus]`` table (root directory, the contract every corpus must meet, default
preparation steps) and one ``[tasks.ID]`` table per corpus with ``shards`` (glob per split, relative to the root),
``raw`` (the source recipe: a ``create_source`` kind plus its arguments) and optional ``prep`` overrides.  The reference
ships the same file as documentation of a lifecycle (raw recipe -> ``prep --task`` -> shards ready -> mixtures use the
task, configs/tasks.toml:1-50) without code behind it; here it is executable:

  ``Registry.status()``           ready (shards found) / buildable (raw material found) per task
  ``Registry.build(task)``        raw -> hygiene -> exact dedup (text) -> quality filter (+ audit) -> exact / near dedup
                                  (tokens) -> tokenise -> shards under the task's directory, contract checked
  ``Registry.check_contract(m)``  a manifest against the corpus contract
  ``Registry.shard_files(task)``  what a loader would read

CLI: ``python -m nmoe_b200.data.cli tasks`` and ``... prep --task ID``.
"""
from __future__ import annotations

import glob as _glob
import hashlib
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Callable, Dict, Iterator, List, Optional

from ..config import load_toml
from .errors import ErrorCode, PipelineError
from .sources import DataSource, Document, create_source

STEPS = ("hygiene", "exact_dedup_text", "hydra_filter", "hydra_audit", "exact_dedup_tokens", "near_dedup_tokens")
_GLOB_CHARS = "*?["


class TaskNotBuildable(PipelineError):
  code = ErrorCode.SOURCE_NOTFOUND


class ContractViolation(PipelineError):
  code = ErrorCode.TOKENIZER_DRIFT


@dataclass
class TaskSpec:
  id: str
  domain: str = "web"
  description: str = ""
  shards: Dict[str, str] = field(default_factory=dict)      # split -> glob relative to the corpus root
  raw: Dict[str, Any] = field(default_factory=dict)
  prep: Dict[str, Any] = field(default_factory=dict)        # defaults merged with the task's overrides

  def shard_dir(self, split: str = "train") -> str:
    """The directory part of the split's pattern: everything before the first component with a wildcard."""
    pat = self.shards.get(split)
    if not pat:
      raise KeyError(f"task {self.id!r} has no '{split}' split; it has {sorted(self.shards)}")
    keep = []
    for part in pat.split("/"):
      if any(c in part for c in _GLOB_CHARS):
        break
      keep.append(part)
    return "/".join(keep)


class _Mapped(DataSource):
  def __init__(self, base: DataSource, fn: Callable[[Iterator[Document]], Iterator[Document]], label: str):
    self.base, self.fn, self.name = base, fn, f"{label}:{base.name}"

  def __iter__(self):
    return self.fn(iter(self.base))


class Registry:
  def __init__(self, spec: Dict[str, Any], path: Optional[Path] = None):
    corpus = spec.get("corpus") or {}
    if "root" not in corpus:
      raise ValueError("the registry needs [corpus] root")
    self.path = path
    self.root = Path(corpus["root"])
    self.contract: Dict[str, Any] = dict(corpus.get("contract") or {})
    self.defaults: Dict[str, Any] = dict(corpus.get("prep_defaults") or {})
    self.tasks: Dict[str, TaskSpec] = {}
    for tid, t in (spec.get("tasks") or {}).items():
      unknown = set(t.get("prep") or {}) - set(STEPS) - {"num_shards", "min_chars"}
      if unknown:
        raise ValueError(f"task {tid!r}: unknown preparation keys {sorted(unknown)}")
      self.tasks[tid] = TaskSpec(tid, t.get("domain", "web"), t.get("description", ""), dict(t.get("shards") or {}),
                                 dict(t.get("raw") or {}), {**self.defaults, **(t.get("prep") or {})})

  @classmethod
  def load(cls, path="configs/tasks.toml") -> "Registry":
    return cls(load_toml(path), Path(path))

  def task(self, tid: str) -> TaskSpec:
    if tid not in self.tasks:
      raise KeyError(f"unknown task {tid!r}; the registry has {sorted(self.tasks)}")
    return self.tasks[tid]

  # -- what exists
  def shard_files(self, tid: str, split: str = "train") -> List[str]:
    pat = self.task(tid).shards.get(split)
    return sorted(_glob.glob(str(self.root / pat), recursive=True)) if pat else []

  def raw_files(self, tid: str) -> Optional[List[str]]:
    """Files of the raw recipe, or None when the recipe is not file-based (a hub dataset) or absent."""
    raw = self.task(tid).raw
    if "glob" in raw:
      return sorted(_glob.glob(str(raw["glob"]), recursive=True))
    for key in ("tar_dir", "html_dir", "paths"):
      if key in raw:
        p = Path(str(raw[key]))
        return sorted(str(x) for x in p.iterdir()) if p.is_dir() else []
    return None

  def status(self) -> List[Dict[str, Any]]:
    rows = []
    for tid, t in sorted(self.tasks.items()):
      shards = self.shard_files(tid) if "train" in t.shards else []
      raw = self.raw_files(tid)
      tokens = None
      man = self.root / t.shard_dir() / "manifest.json" if t.shards.get("train") else None
      if man is not None and man.exists():
        from .sinks import load_manifest
        tokens = load_manifest(man).total_tokens
      rows.append({"task": tid, "domain": t.domain, "ready": bool(shards), "shards": len(shards), "tokens": tokens,
                   "buildable": bool(t.raw) and (raw is None or len(raw) > 0), "raw_files": None if raw is None else len(raw),
                   "raw_kind": t.raw.get("kind")})
    return rows

  # -- contract
  def check_contract(self, manifest) -> None:
    c = self.contract
    bad = []
    for key in ("tokenizer", "vocab_size", "eos_token_id", "dtype"):
      if key in c and getattr(manifest, key, None) != c[key]:
        bad.append(f"{key}: corpus wants {c[key]!r}, the dataset has {getattr(manifest, key, None)!r}")
    if bad:
      raise ContractViolation(f"dataset {manifest.dataset!r} breaks the corpus contract: " + "; ".join(bad))

  # -- building
  def source(self, tid: str) -> DataSource:
    t = self.task(tid)
    if not t.raw or "kind" not in t.raw:
      raise TaskNotBuildable(f"task {tid!r} has no [raw] recipe: it cannot be built from this registry")
    kw = {k: v for k, v in t.raw.items() if k != "kind"}
    if "glob" in kw:
      kw["paths"] = kw.pop("glob")
    if t.raw["kind"] == "arxiv_s3":            # the reference's name for the bulk-tar source
      return create_source("arxiv_tars", **kw)
    return create_source(t.raw["kind"], **kw)

  def pipeline(self, tid: str, src: DataSource, *, grader=None, tau_keep: float = 0.0, audit_dir: Optional[Path] = None,
               tokenizer: Optional[str] = None, stats: Optional[dict] = None) -> DataSource:
    """The task's preparation steps as wrappers around ``src``, in the registry's order."""
    from .dedup import dedup_exact, stream_near_dedup
    from .sources import AuditedSource, FilteredSource, ScoringSource
    from .transforms import normalize_text, tokenize
    p = self.task(tid).prep
    st = stats if stats is not None else {}
    if p.get("hygiene"):
      min_chars = int(p.get("min_chars", 32))
      def clean(docs):
        for d in docs:
          t = normalize_text(d.text)
          t = "".join(ch for ch in t if ch >= " " or ch in "\n\t")
          if len(t.strip()) >= min_chars:
            yield Document(d.doc_id, t, d.metadata)
          else:
            st["hygiene_dropped"] = st.get("hygiene_dropped", 0) + 1
      src = _Mapped(src, clean, "clean")
    if p.get("exact_dedup_text"):
      src = _Mapped(src, dedup_exact, "dedup")
    if p.get("hydra_filter") or (p.get("hydra_audit") and audit_dir is not None):
      if grader is None:
        if p.get("hydra_filter"):
          raise TaskNotBuildable(f"task {tid!r} filters by quality: give a grading model (--checkpoint / --heads-dir) or --no-hydra")
      else:
        scored = ScoringSource(src, grader)
        thr = tau_keep if p.get("hydra_filter") else None
        src = AuditedSource(scored, audit_dir, thr) if (p.get("hydra_audit") and audit_dir is not None) else \
            (FilteredSource(scored, tau_keep) if thr is not None else scored)
    if p.get("exact_dedup_tokens"):
      tok = tokenizer or self.contract.get("tokenizer", "o200k_harmony")
      def by_tokens(docs):
        seen = set()
        for d in docs:
          h = hashlib.blake2b(b"".join(int(t).to_bytes(4, "little") for t in tokenize(d.text, tok)), digest_size=16).digest()
          if h not in seen:
            seen.add(h)
            yield d
      src = _Mapped(src, by_tokens, "dedup_tokens")
    if p.get("near_dedup_tokens"):
      src = _Mapped(src, lambda docs: stream_near_dedup(docs, threshold=0.8), "near_dedup")
    return src

  def build(self, tid: str, split: str = "train", *, grader=None, tau_keep: float = 0.0, no_hydra: bool = False,
            max_documents: Optional[int] = None, tokenizer: Optional[str] = None, num_shards: Optional[int] = None,
            source: Optional[DataSource] = None, print_fn: Callable = print):
    """Build the task's shards for ``split`` and check the result against the corpus contract.  Returns the manifest."""
    from .prep import PrepConfig, PrepPipeline
    t = self.task(tid)
    if no_hydra:
      t = TaskSpec(t.id, t.domain, t.description, t.shards, t.raw, {**t.prep, "hydra_filter": False, "hydra_audit": False})
      self.tasks[tid] = t
    out = self.root / t.shard_dir(split)
    src = self.pipeline(tid, source or self.source(tid), grader=grader, tau_keep=tau_keep, audit_dir=out / "hydra_audit",
                        tokenizer=tokenizer)
    cfg = PrepConfig(output_dir=str(out), dataset=tid, version="v1", tokenizer=tokenizer or self.contract.get("tokenizer", "o200k_harmony"),
                     num_shards=int(num_shards or t.prep.get("num_shards", 64)), max_documents=max_documents,
                     source_info={"task": tid, "raw": t.raw, "prep": {k: bool(t.prep.get(k)) for k in STEPS}})
    m = PrepPipeline(src, cfg, print_fn=print_fn).run()
    if tokenizer is None:
      self.check_contract(m)
    print_fn(f"[registry] task {tid}: {m.total_documents:,} documents, {m.total_tokens:,} tokens -> {out}")
    return m
