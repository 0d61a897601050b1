"""Read-only dataset browser behind the dashboard's ``/api/datasets/*`` routes (reference: nviz/lib/server/datasets.ts,
datasets_inspect.ts, datasets_pipeline.ts and nviz/app/api/datasets/*/route.ts).

Every path is relative to a root directory (``NVIZ_DATASETS_DIR``, default ``/data``); a path that resolves outside the
root is refused.  Routes:

  /api/datasets?path=P                         directory listing (dirs first), sizes and mtimes
  /api/datasets/preview?path=P[&bytes=N]       head of a file as text (or a hex dump when it is binary)
  /api/datasets/meta?path=P                    what the path is: token shard, index, manifest, flow directory, ...
  /api/datasets/manifest?path=DIR[&limit=N]    manifest.json of a prepared dataset with the first N shard records
  /api/datasets/shard/stats?path=SHARD         tokens, documents, document-length and token-id statistics
  /api/datasets/shard/window?path=SHARD&offset=O&length=L[&tokenizer=T]   token ids (and text when decodable)
  /api/datasets/index/header?path=IDX          number of documents, length statistics from the (start, end) pairs
  /api/datasets/index/doc?path=IDX&doc=I[&tokenizer=T]   one document's span and tokens
  /api/datasets/pipeline?path=DIR              a flow directory: stages / sources, shard counts, token totals
"""
from __future__ import annotations

import json
import os
from pathlib import Path
from typing import Dict, List, Optional

import numpy as np

from ..data import inspect as I
from ..data.index import HEADER_SIZE, IndexReader, index_path_for_shard, unpack_header


class DatasetPathError(ValueError):
  pass


def datasets_root() -> Path:
  return Path(os.environ.get("NVIZ_DATASETS_DIR", "/data")).resolve()


def safe_resolve(rel: str, root: Optional[Path] = None) -> Path:
  root = (root or datasets_root()).resolve()
  target = (root / (rel or ".")).resolve()
  if target != root and root not in target.parents:
    raise DatasetPathError("path escapes the datasets directory")
  return target


def list_dir(rel: str, root: Optional[Path] = None) -> Dict:
  d = safe_resolve(rel, root)
  if not d.is_dir():
    raise DatasetPathError("not a directory")
  entries = []
  for e in d.iterdir():
    try:
      st = e.stat()
    except OSError:
      continue
    entries.append({"name": e.name, "kind": "dir" if e.is_dir() else "file", "size": int(st.st_size),
                    "mtime_ms": int(st.st_mtime * 1000)})
  entries.sort(key=lambda x: (x["kind"] != "dir", x["name"]))
  return {"path": rel or "", "entries": entries}


def preview_file(rel: str, max_bytes: int = 64 * 1024, root: Optional[Path] = None) -> Dict:
  p = safe_resolve(rel, root)
  if not p.is_file():
    raise DatasetPathError("not a file")
  cap = max(1024, min(int(max_bytes), 1 << 20))
  with open(p, "rb") as f:
    buf = f.read(cap)
  printable = sum(1 for b in buf if b in (9, 10, 13) or 32 <= b <= 126)
  if not buf or printable / len(buf) >= 0.8:
    return {"path": rel, "bytes": len(buf), "text": buf.decode("utf-8", errors="replace")}
  return {"path": rel, "bytes": len(buf), "hex": buf[:256].hex(" ")}


def meta(rel: str, root: Optional[Path] = None) -> Dict:
  p = safe_resolve(rel, root)
  out = {"path": rel, "exists": p.exists(), "kind": "missing"}
  if not p.exists():
    return out
  if p.is_dir():
    out["kind"] = "dir"
    out["has_manifest"] = (p / "manifest.json").exists()
    out["npy_shards"] = sum(1 for _ in p.glob("*.npy"))
    out["is_flow_dir"] = any((c / "manifest.json").exists() for c in p.iterdir() if c.is_dir())
    return out
  out["size"] = p.stat().st_size
  if p.suffix == ".npy":
    out["kind"] = "token_shard"
    out["has_index"] = index_path_for_shard(p).exists()
  elif p.suffix == ".idx":
    out["kind"] = "index"
  elif p.name == "manifest.json":
    out["kind"] = "manifest"
  else:
    out["kind"] = "file"
  return out


def manifest_preview(rel_dir: str, limit: int = 200, root: Optional[Path] = None) -> Dict:
  d = safe_resolve(rel_dir, root)
  mp = d / "manifest.json" if d.is_dir() else d
  if not mp.exists():
    raise DatasetPathError("no manifest.json here")
  m = json.loads(mp.read_text())
  shards = m.get("shards", [])
  head = {k: v for k, v in m.items() if k != "shards"}
  head["num_shards_listed"] = len(shards)
  return {"path": rel_dir, "manifest": head, "shards": shards[:max(0, int(limit))]}


def shard_stats(rel: str, root: Optional[Path] = None, sample: int = 1 << 22) -> Dict:
  p = safe_resolve(rel, root)
  out = I.shard_stats(p)
  out["path"] = rel
  t = np.load(p, mmap_mode="r")
  n = int(t.shape[0])
  if n:
    head = np.asarray(t[:min(n, sample)]).astype(np.int64)
    uniq = np.unique(head)
    out.update({"sampled_tokens": int(head.size), "unique_token_ids_in_sample": int(uniq.size),
                "min_token_id": int(head.min())})
  return out


def token_window(rel: str, offset: int, length: int, tokenizer: Optional[str] = None, root: Optional[Path] = None) -> Dict:
  p = safe_resolve(rel, root)
  length = max(0, min(int(length), 65536))
  out = I.shard_window(p, max(0, int(offset)), length, tokenizer)
  out["path"] = rel
  return out


def index_header(rel: str, root: Optional[Path] = None) -> Dict:
  p = safe_resolve(rel, root)
  with open(p, "rb") as f:
    n = unpack_header(f.read(HEADER_SIZE))
  out = {"path": rel, "documents": n, "bytes": p.stat().st_size}
  if n:
    b = IndexReader(p).to_array()
    lens = (b[:, 1] - b[:, 0]).astype(np.int64)
    out.update({"doc_len_mean": float(lens.mean()), "doc_len_p50": float(np.percentile(lens, 50)),
                "doc_len_p99": float(np.percentile(lens, 99)), "doc_len_max": int(lens.max()),
                "tokens_covered": int(lens.sum())})
  return out


def index_doc(rel: str, doc: int, tokenizer: Optional[str] = None, max_tokens: int = 8192, root: Optional[Path] = None) -> Dict:
  p = safe_resolve(rel, root)
  s, e = IndexReader(p).get_document(int(doc))
  out = {"path": rel, "doc": int(doc), "start": s, "end": e, "tokens": e - s}
  shard = p.with_suffix(".npy")
  if shard.exists():
    w = I.shard_window(shard, s, min(e - s, max_tokens), tokenizer)
    out.update({k: v for k, v in w.items() if k in ("ids", "text", "text_error")})
  return out


def pipeline_inspect(rel_dir: str, root: Optional[Path] = None) -> Dict:
  """A flow directory (one sub-directory per source, each a prepared dataset with a manifest)."""
  d = safe_resolve(rel_dir, root)
  if not d.is_dir():
    raise DatasetPathError("not a directory")
  sources: List[Dict] = []
  for c in sorted(x for x in d.iterdir() if x.is_dir()):
    mp = c / "manifest.json"
    rec = {"source": c.name, "has_manifest": mp.exists(), "npy_shards": sum(1 for _ in c.glob("*.npy")),
           "idx_files": sum(1 for _ in c.glob("*.idx"))}
    if mp.exists():
      try:
        m = json.loads(mp.read_text())
        rec.update({"dataset": m.get("dataset"), "version": m.get("version"), "tokenizer": m.get("tokenizer"),
                    "total_tokens": m.get("total_tokens"), "total_documents": m.get("total_documents"),
                    "num_shards": m.get("num_shards")})
      except (OSError, ValueError) as e:
        rec["manifest_error"] = str(e)
    sources.append(rec)
  return {"path": rel_dir, "sources": sources,
          "total_tokens": sum(int(s.get("total_tokens") or 0) for s in sources)}
