"""Run dashboard: a read-only HTTP service over the per-rank metric files and the experiments DB.

  python -m nmoe_b200.viz.server --metrics-dir /data/metrics --experiments-db /data/experiments.db --port 3000

Endpoints.  Paths, query parameters and the JSON keys named here are those of the reference dashboard's routes
(nviz/app/api/*/route.ts, client types in nviz/lib/api.ts), so a front end written against one works with the other:

  GET /api/health                                 -> {ok, runs}
  GET /api/runs                                   -> {runs: [{run, last_ts, last_step, ranks, status?, experiment_id?,
                                                     started_at?, ended_at?}]}: metric files merged with the
                                                     experiments DB (a run known only to the DB has last_step 0),
                                                     newest first
  GET /api/tags?run=R                             -> {run, tags: [...]}
  GET /api/series?run=R&tag=T[&points=N][&rank=r] -> {run, tag, series: [{step, ts_ms, value}]}  (LTTB, <= N, default 1000)
  GET /api/summary?run=R                          -> {run, summary: {tag: latest value}, steps: {tag: step}} without
                                                     per-rank timers, per-GPU and per-layer tags
  GET /api/gpu?run=R                              -> {run, gpus: [{index, <metric>: value}], agg: {"gpu_agg/*": value}}
  GET /api/router?run=R                           -> {run, layers: [{idx, cv, entropy, max_load, bias_range,
                                                     experts_active}], agg: {"router_agg/*": value}}
  GET /api/experiments                            -> {experiments: [{id, name, project, description, created_at,
                                                     runs_total, runs_running, runs_completed, runs_failed,
                                                     runs_killed, last_started_at}]}
  GET /api/experiments/runs[?experiment_id=E][&limit=N] -> {runs: [run row + last_ts, last_step]}
  GET /api/experiments/run?run=R                  -> {run: row} or 404
  GET /api/datasets[/preview|/meta|/manifest|/shard/stats|/shard/window|/index/header|/index/doc|/pipeline]?path=P
                                                  -> read-only dataset browser confined to NVIZ_DATASETS_DIR (viz/datasets.py)
  GET /, /static/*                                -> the dashboard page (viz/static/): runs, charts with run comparison,
                                                     GPU monitor, router heat map, experiments table, dataset browser

All ``rank_*.duckdb`` / ``rank_*.sqlite`` files of a run are opened read-only and merged; when a
(tag, step) appears in several rank files the newest ``ts_ms`` wins (the reference does the same
with a window function, nviz/lib/server/duckdb.ts:68-194).  Only the standard library is needed
unless the files are DuckDB files.
"""
from __future__ import annotations

import argparse
import json
import re
import sqlite3
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from pathlib import Path
from typing import Dict, Iterable, List, Optional, Sequence, Tuple
from urllib.parse import parse_qs, urlparse

Point = Tuple[int, float]


def lttb(points: Sequence[Point], n_out: int) -> List[Point]:
  """Largest-Triangle-Three-Buckets down-sampling (nviz/app/api/series/route.ts:6-37): keeps the
  first and last point and, per bucket, the point spanning the largest triangle with the previous
  pick and the next bucket's mean."""
  n = len(points)
  if n_out >= n or n_out < 3:
    return list(points)
  out = [points[0]]
  every = (n - 2) / (n_out - 2)
  a = 0
  for i in range(n_out - 2):
    lo = int((i + 1) * every) + 1
    hi = min(int((i + 2) * every) + 1, n)
    nxt = points[lo:hi] or [points[-1]]
    ax = sum(p[0] for p in nxt) / len(nxt)
    ay = sum(p[1] for p in nxt) / len(nxt)
    b_lo = int(i * every) + 1
    b_hi = min(int((i + 1) * every) + 1, n - 1)
    best, best_area = b_lo, -1.0
    px, py = points[a]
    for j in range(b_lo, max(b_hi, b_lo + 1)):
      area = abs((px - ax) * (points[j][1] - py) - (px - points[j][0]) * (ay - py))
      if area > best_area:
        best, best_area = j, area
    out.append(points[best])
    a = best
  out.append(points[-1])
  return out


class MetricStore:
  """Read-only view of ``{metrics_dir}/{run}/rank_*.{sqlite,duckdb}``."""

  def __init__(self, metrics_dir: str):
    self.root = Path(metrics_dir)

  def runs(self) -> List[str]:
    if not self.root.is_dir():
      return []
    return sorted(p.name for p in self.root.iterdir() if p.is_dir() and any(p.glob("rank_*.*")))

  def _files(self, run: str, rank: Optional[int] = None) -> List[Path]:
    d = self.root / run
    if not re.fullmatch(r"[\w.\-]+", run) or not d.is_dir():
      return []
    pat = "rank_*" if rank is None else f"rank_{int(rank)}"
    return sorted(p for p in d.glob(pat + ".*") if p.suffix in (".sqlite", ".duckdb"))

  @staticmethod
  def _query(path: Path, sql: str, args: Tuple) -> List[Tuple]:
    if path.suffix == ".duckdb":
      import duckdb  # type: ignore
      con = duckdb.connect(str(path), read_only=True)
      try:
        return con.execute(sql, list(args)).fetchall()
      finally:
        con.close()
    con = sqlite3.connect(f"file:{path}?mode=ro", uri=True, timeout=5.0)
    try:
      return con.execute(sql, args).fetchall()
    finally:
      con.close()

  def _merged(self, run: str, where: str, args: Tuple, rank: Optional[int] = None) -> Dict[Tuple[str, int], Tuple[int, float]]:
    """(tag, step) -> (ts_ms, value), newest ts wins across rank files."""
    best: Dict[Tuple[str, int], Tuple[int, float]] = {}
    for f in self._files(run, rank):
      try:
        rows = self._query(f, f"SELECT tag, step, ts_ms, value FROM metrics WHERE run = ? AND {where}", (run,) + args)
      except (sqlite3.Error, ImportError):
        continue
      for tag, step, ts, val in rows:
        k = (tag, int(step))
        if k not in best or ts > best[k][0]:
          best[k] = (int(ts), float(val))
    return best

  def series(self, run: str, tag: str, points: int = 1000, rank: Optional[int] = None) -> List[Point]:
    return [(s, v) for s, _, v in self.series_ts(run, tag, points, rank)]

  def series_ts(self, run: str, tag: str, points: int = 1000, rank: Optional[int] = None) -> List[Tuple[int, int, float]]:
    """(step, ts_ms, value) of a tag, down-sampled on (step, value)."""
    m = self._merged(run, "tag = ?", (tag,), rank)
    ts = {step: t for (_, step), (t, _) in m.items()}
    pts = sorted((step, v) for (_, step), (_, v) in m.items())
    return [(s, ts[s], v) for s, v in lttb(pts, points)]

  def tags(self, run: str) -> List[str]:
    out = set()
    for f in self._files(run):
      try:
        out.update(r[0] for r in self._query(f, "SELECT DISTINCT tag FROM metrics WHERE run = ?", (run,)))
      except (sqlite3.Error, ImportError):
        continue
    return sorted(out)

  def latest(self, run: str, like: str) -> Dict[str, Tuple[int, float]]:
    """tag -> (step, value) at each tag's last step, for tags matching the SQL LIKE pattern."""
    m = self._merged(run, "tag LIKE ?", (like,))
    out: Dict[str, Tuple[int, float]] = {}
    for (tag, step), (_, v) in m.items():
      if tag not in out or step > out[tag][0]:
        out[tag] = (step, v)
    return out

  def run_info(self, run: str) -> dict:
    files = self._files(run)
    last_step, last_ts = -1, 0
    for f in files:
      try:
        rows = self._query(f, "SELECT MAX(step), MAX(ts_ms) FROM metrics WHERE run = ?", (run,))
      except (sqlite3.Error, ImportError):
        continue
      if rows and rows[0][0] is not None:
        last_step = max(last_step, int(rows[0][0]))
        last_ts = max(last_ts, int(rows[0][1]))
    return {"run": run, "ranks": len(files), "last_step": max(last_step, 0), "last_ts": last_ts}


def group_gpu(latest: Dict[str, Tuple[int, float]]) -> Tuple[List[dict], Dict[str, float]]:
  """Latest ``gpu/{i}/{metric}`` values as one record per GPU index, and the ``gpu_agg/*`` values by full tag."""
  by_idx: Dict[int, dict] = {}
  agg: Dict[str, float] = {}
  for tag, (_, v) in latest.items():
    m = re.fullmatch(r"gpu/(\d+)/(\w+)", tag)
    if m:
      by_idx.setdefault(int(m.group(1)), {"index": int(m.group(1))})[m.group(2)] = v
    elif tag.startswith("gpu_agg/"):
      agg[tag] = v
  return [by_idx[i] for i in sorted(by_idx)], agg


def group_router(latest: Dict[str, Tuple[int, float]]) -> Tuple[List[dict], Dict[str, float]]:
  """Latest ``router/layer_NN/{metric}`` values as one record per layer, and the ``router_agg/*`` values by full tag."""
  by_idx: Dict[int, dict] = {}
  agg: Dict[str, float] = {}
  for tag, (_, v) in latest.items():
    m = re.fullmatch(r"router/layer_(\d+)/(\w+)", tag)
    if m:
      by_idx.setdefault(int(m.group(1)), {"idx": int(m.group(1))})[m.group(2)] = v
    elif tag.startswith("router_agg/"):
      agg[tag] = v
  return [by_idx[i] for i in sorted(by_idx)], agg


class ExperimentsView:
  """Read-only queries on the experiments database (nviz/lib/server/experiments.ts:106-290).  Every call opens the
  file afresh in read-only mode, so a training job that is writing to it is never blocked; a missing or unreadable
  database reads as empty."""

  RUN_COLS = ("id", "experiment_id", "status", "started_at", "ended_at", "git_hash", "git_dirty", "config_json", "results_json")

  def __init__(self, db_path: Optional[str]):
    self.path = db_path

  def _rows(self, sql: str, args: Tuple = ()) -> List[sqlite3.Row]:
    if not self.path or not Path(self.path).exists():
      return []
    try:
      con = sqlite3.connect(f"file:{self.path}?mode=ro", uri=True, timeout=5.0)
    except sqlite3.Error:
      return []
    con.row_factory = sqlite3.Row
    try:
      return con.execute(sql, args).fetchall()
    except sqlite3.Error:
      return []
    finally:
      con.close()

  def _run_row(self, r: sqlite3.Row) -> dict:
    d = {k: r[k] for k in self.RUN_COLS}
    d["run"] = d.pop("id")
    return d

  def run_states(self) -> List[dict]:
    return [{"run": r["id"], "experiment_id": r["experiment_id"], "status": r["status"], "started_at": r["started_at"],
             "ended_at": r["ended_at"]} for r in self._rows("SELECT id, experiment_id, status, started_at, ended_at FROM runs")]

  def summaries(self) -> List[dict]:
    exps = self._rows("SELECT * FROM experiments ORDER BY created_at DESC, id")
    out = []
    for e in exps:
      keys = e.keys()
      d = {"id": e["id"], "name": e["name"] if "name" in keys else e["id"], "project": e["project"] if "project" in keys else "default",
           "description": e["description"], "created_at": e["created_at"]}
      counts = {r["status"]: r["n"] for r in self._rows("SELECT status, COUNT(*) AS n FROM runs WHERE experiment_id = ? GROUP BY status", (e["id"],))}
      d["runs_total"] = sum(counts.values())
      for st in ("running", "completed", "failed", "killed"):
        d[f"runs_{st}"] = counts.get(st, 0)
      last = self._rows("SELECT MAX(started_at) AS t FROM runs WHERE experiment_id = ?", (e["id"],))
      d["last_started_at"] = last[0]["t"] if last else None
      out.append(d)
    return out

  def runs(self, experiment_id: Optional[str] = None, limit: int = 200) -> List[dict]:
    limit = max(1, min(int(limit), 2000))
    cols = ", ".join(self.RUN_COLS)
    if experiment_id:
      rows = self._rows(f"SELECT {cols} FROM runs WHERE experiment_id = ? ORDER BY started_at DESC, id LIMIT ?", (experiment_id, limit))
    else:
      rows = self._rows(f"SELECT {cols} FROM runs ORDER BY started_at DESC, id LIMIT ?", (limit,))
    return [self._run_row(r) for r in rows]

  def run(self, run_id: str) -> Optional[dict]:
    rows = self._rows(f"SELECT {', '.join(self.RUN_COLS)} FROM runs WHERE id = ?", (run_id,))
    return self._run_row(rows[0]) if rows else None


def merged_runs(store: MetricStore, exps: ExperimentsView) -> List[dict]:
  """Runs that have metric files, joined with the runs the experiments database knows (nviz/app/api/runs/route.ts:5-43);
  newest activity first, then newest start, then highest step, then name."""
  by_id: Dict[str, dict] = {r: store.run_info(r) for r in store.runs()}
  for st in exps.run_states():
    cur = by_id.setdefault(st["run"], {"run": st["run"], "ranks": 0, "last_ts": 0, "last_step": 0})
    cur.update({k: st[k] for k in ("experiment_id", "status", "started_at", "ended_at")})
  runs = list(by_id.values())
  runs.sort(key=lambda r: r["run"])
  runs.sort(key=lambda r: (r.get("last_ts") or 0, str(r.get("started_at") or ""), r.get("last_step") or 0), reverse=True)
  return runs


STATIC_DIR = Path(__file__).resolve().parent / "static"
_CTYPES = {".html": "text/html; charset=utf-8", ".js": "text/javascript; charset=utf-8", ".css": "text/css; charset=utf-8",
           ".svg": "image/svg+xml", ".json": "application/json"}


def static_file(rel: str) -> Optional[Tuple[bytes, str]]:
  """A file of the dashboard page; names are matched against the directory listing, so no path can leave it."""
  name = rel.strip("/") or "index.html"
  for f in STATIC_DIR.iterdir() if STATIC_DIR.is_dir() else ():
    if f.is_file() and f.name == name and f.suffix in _CTYPES:
      return f.read_bytes(), _CTYPES[f.suffix]
  return None


def make_handler(store: MetricStore, exp_db: Optional[str]):
  exps = ExperimentsView(exp_db)

  class Handler(BaseHTTPRequestHandler):
    def log_message(self, fmt, *args):   # quiet
      pass

    def _send(self, code: int, body, ctype: str = "application/json") -> None:
      data = body if isinstance(body, bytes) else body.encode() if isinstance(body, str) else json.dumps(body).encode()
      self.send_response(code)
      self.send_header("Content-Type", ctype)
      self.send_header("Cache-Control", "private, max-age=2")
      self.send_header("Content-Length", str(len(data)))
      self.end_headers()
      self.wfile.write(data)

    def _datasets(self, what: str, q: Dict[str, str]):
      """Read-only dataset browser (viz/datasets.py); every path is confined to NVIZ_DATASETS_DIR.  Query parameters
      take the names of the reference's routes (``max_bytes``, ``limit_shards``, ``shard_path`` / ``doc_idx`` /
      ``max_tokens``) as well as the shorter ones this server started with."""
      from . import datasets as D
      path = q.get("path", "")
      try:
        if what == "":
          return self._send(200, D.list_dir(path))
        if what == "preview":
          return self._send(200, D.preview_file(path, int(q.get("max_bytes", q.get("bytes", str(64 * 1024))))))
        if what == "meta":
          return self._send(200, D.meta(path))
        if what == "manifest":
          return self._send(200, D.manifest_preview(path, int(q.get("limit_shards", q.get("limit", "200")))))
        if what == "shard/stats":
          return self._send(200, D.shard_stats(path))
        if what == "shard/window":
          return self._send(200, D.token_window(path, int(q.get("offset", "0")), int(q.get("length", "256")),
                                                q.get("tokenizer")))
        if what == "index/header":
          return self._send(200, D.index_header(path))
        if what == "index/doc":
          if not path and q.get("shard_path"):      # the document may be named by its shard instead of its index file
            path = re.sub(r"\.npy$", ".idx", q["shard_path"])
          return self._send(200, D.index_doc(path, int(q.get("doc_idx", q.get("doc", "0"))), q.get("tokenizer"),
                                             int(q.get("max_tokens", "8192"))))
        if what == "pipeline":
          return self._send(200, D.pipeline_inspect(path))
        return self._send(404, {"error": "not found"})
      except D.DatasetPathError as e:
        return self._send(400, {"error": str(e)})
      except (FileNotFoundError, IndexError) as e:
        return self._send(404, {"error": str(e)})

    def do_GET(self):
      u = urlparse(self.path)
      q = {k: v[0] for k, v in parse_qs(u.query).items()}
      try:
        if u.path == "/" or u.path.startswith("/static/"):
          hit = static_file("" if u.path == "/" else u.path[len("/static/"):])
          if hit is None:
            return self._send(404, {"error": "not found"})
          return self._send(200, hit[0], hit[1])
        if u.path == "/api/health":
          return self._send(200, {"ok": True, "runs": len(store.runs())})
        if u.path == "/api/runs":
          return self._send(200, {"runs": merged_runs(store, exps)})
        if u.path == "/api/experiments":
          return self._send(200, {"experiments": exps.summaries()})
        if u.path == "/api/experiments/runs":
          info = {r: store.run_info(r) for r in store.runs()}
          rows = exps.runs(q.get("experiment_id") or None, int(q.get("limit", "200")))
          for r in rows:
            m = info.get(r["run"], {})
            r["last_ts"], r["last_step"] = m.get("last_ts", 0), m.get("last_step", 0)
          return self._send(200, {"runs": rows})
        if u.path == "/api/experiments/run":
          if not q.get("run"):
            return self._send(400, {"error": "Missing 'run'"})
          row = exps.run(q["run"])
          return self._send(200, {"run": row}) if row else self._send(404, {"error": "Not found"})
        if u.path == "/api/datasets" or u.path.startswith("/api/datasets/"):
          return self._datasets(u.path[len("/api/datasets"):].strip("/"), q)
        run = q.get("run", "")
        if u.path.startswith("/api/") and not run:
          return self._send(400, {"error": "Missing 'run'"})
        if u.path.startswith("/api/") and run not in store.runs():
          return self._send(404, {"error": f"unknown run {run!r}"})
        if u.path == "/api/tags":
          return self._send(200, {"run": run, "tags": store.tags(run)})
        if u.path == "/api/series":
          if "tag" not in q:
            return self._send(400, {"error": "Missing 'run' or 'tag'"})
          n = max(3, min(int(q.get("points", "1000")), 5000))
          rank = int(q["rank"]) if "rank" in q else None
          pts = store.series_ts(run, q["tag"], n, rank)
          return self._send(200, {"run": run, "tag": q["tag"], "series": [{"step": s, "ts_ms": t, "value": v} for s, t, v in pts]})
        if u.path == "/api/summary":
          lat = {t: sv for t, sv in sorted(store.latest(run, "%").items())
                 if not t.startswith(("time_ms/", "gpu/", "router/layer_"))}
          return self._send(200, {"run": run, "summary": {t: v for t, (_, v) in lat.items()}, "steps": {t: s for t, (s, _) in lat.items()}})
        if u.path == "/api/gpu":
          gpus, agg = group_gpu(store.latest(run, "gpu%"))
          return self._send(200, {"run": run, "gpus": gpus, "agg": agg})
        if u.path == "/api/router":
          layers, agg = group_router(store.latest(run, "router%"))
          return self._send(200, {"run": run, "layers": layers, "agg": agg})
        return self._send(404, {"error": "not found"})
      except (ValueError, OSError) as e:
        return self._send(400, {"error": str(e)})

  return Handler


def serve(metrics_dir: str, experiments_db: Optional[str], host: str = "127.0.0.1", port: int = 3000) -> ThreadingHTTPServer:
  srv = ThreadingHTTPServer((host, port), make_handler(MetricStore(metrics_dir), experiments_db))
  return srv


def main(argv: Optional[Iterable[str]] = None) -> None:
  ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
  ap.add_argument("--metrics-dir", required=True)
  ap.add_argument("--experiments-db", default=None)
  ap.add_argument("--host", default="127.0.0.1")
  ap.add_argument("--port", type=int, default=3000)
  a = ap.parse_args(list(argv) if argv is not None else None)
  srv = serve(a.metrics_dir, a.experiments_db, a.host, a.port)
  print(f"serving {a.metrics_dir} on http://{a.host}:{srv.server_address[1]}")
  try:
    srv.serve_forever()
  except KeyboardInterrupt:
    pass
  finally:
    srv.server_close()


if __name__ == "__main__":
  main()
