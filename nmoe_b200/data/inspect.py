"""Human-readable views of shards and indices (nmoe/data/inspect.py): header, per-shard statistics,
a decoded window of tokens, one document."""
from __future__ import annotations

from pathlib import Path
from typing import Dict, Optional

import numpy as np

from .index import IndexReader, index_path_for_shard
from .sinks import load_manifest
from .transforms import get_tokenizer


def shard_stats(shard: Path) -> Dict:
  t = np.load(shard, mmap_mode="r")
  out = {"path": str(shard), "tokens": int(t.shape[0]), "dtype": str(t.dtype)}
  ip = index_path_for_shard(Path(shard))
  if ip.exists():
    b = IndexReader(ip).to_array()
    lens = (b[:, 1] - b[:, 0]).astype(np.int64)
    out.update({"documents": int(len(b)), "doc_len_mean": float(lens.mean()) if len(b) else 0.0,
                "doc_len_max": int(lens.max()) if len(b) else 0, "doc_len_min": int(lens.min()) if len(b) else 0})
  if t.shape[0]:
    out["max_token_id"] = int(np.asarray(t).max())
  return out


def shard_window(shard: Path, start: int, length: int, tokenizer: Optional[str] = None) -> Dict:
  t = np.load(shard, mmap_mode="r")
  ids = np.asarray(t[start:start + length]).astype(np.int64).tolist()
  out = {"start": start, "ids": ids}
  if tokenizer:
    try:
      out["text"] = get_tokenizer(tokenizer).decode(ids)
    except Exception as e:  # vocabulary file not available offline
      out["text_error"] = str(e)
  return out


def document(shard: Path, doc_idx: int, tokenizer: Optional[str] = None) -> Dict:
  s, e = IndexReader(index_path_for_shard(Path(shard))).get_document(doc_idx)
  out = shard_window(shard, s, e - s, tokenizer)
  out["doc"] = doc_idx
  return out


def dataset_summary(directory: Path) -> Dict:
  m = load_manifest(directory)
  return {"dataset": m.dataset, "version": m.version, "tokenizer": m.tokenizer, "total_tokens": m.total_tokens,
          "total_documents": m.total_documents, "num_shards": m.num_shards,
          "shards": [shard_stats(Path(directory) / s.path) for s in m.shards[:8]]}
