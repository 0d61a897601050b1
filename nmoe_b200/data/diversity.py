"""Embedding clustering for corpus coverage (nmoe/data/diversity.py:15-96): mini-batch k-means and
coverage statistics (cluster occupancy entropy, max share, empty clusters)."""
from __future__ import annotations

from typing import Dict, Tuple

import numpy as np


def cluster_embeddings(x: np.ndarray, k: int, iters: int = 50, batch: int = 1024, seed: int = 0) -> Tuple[np.ndarray, np.ndarray]:
  """Mini-batch k-means.  Returns (centroids [k,d], assignment [n])."""
  rng = np.random.default_rng(seed)
  n = x.shape[0]
  k = min(k, n)
  cent = x[rng.choice(n, size=k, replace=False)].astype(np.float64).copy()
  counts = np.zeros(k)
  for _ in range(iters):
    b = x[rng.choice(n, size=min(batch, n), replace=False)]
    d = ((b[:, None, :] - cent[None]) ** 2).sum(-1)
    a = d.argmin(1)
    for j in np.unique(a):
      pts = b[a == j]
      counts[j] += len(pts)
      lr = len(pts) / counts[j]
      cent[j] = (1 - lr) * cent[j] + lr * pts.mean(0)
  assign = np.concatenate([((x[i:i + 8192, None, :] - cent[None]) ** 2).sum(-1).argmin(1) for i in range(0, n, 8192)])
  return cent, assign


def coverage_metrics(assign: np.ndarray, k: int) -> Dict[str, float]:
  c = np.bincount(assign, minlength=k).astype(np.float64)
  p = c / max(1.0, c.sum())
  nz = p[p > 0]
  ent = float(-(nz * np.log(nz)).sum())
  return {"entropy": ent, "normalized_entropy": ent / np.log(k) if k > 1 else 1.0, "max_share": float(p.max()),
          "empty_clusters": float((c == 0).sum()), "clusters": float(k)}
