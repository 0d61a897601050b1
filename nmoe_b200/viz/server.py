"""Run dashboard: a read-only HTTP service over the per-rank metric files and the experiments DB.

  python -m nmoe_b200.viz.server --metrics-dir /data/metrics --experiments-db /data/experiments.db --port 3000

Endpoints (same contract as the reference dashboard, nviz/app/api/*/route.ts):

  GET /api/health
  GET /api/runs                                   -> [{run, ranks, last_step, last_ts_ms}]
  GET /api/series?run=R&tag=T[&points=N][&rank=r] -> {run, tag, points:[[step,value],...]}  (LTTB down-sampled, <= N, default 1000)
  GET /api/summary?run=R                          -> latest value of every non-per-rank tag
  GET /api/gpu?run=R                              -> latest gpu/{i}/* telemetry grouped by GPU index
  GET /api/router?run=R                           -> latest router/layer_NN/* and router_agg/* grouped by layer
  GET /api/experiments                            -> experiments with their runs (config, git hash, status, results)
  GET /api/datasets[/preview|/meta|/manifest|/shard/stats|/shard/window|/index/header|/index/doc|/pipeline]?path=P
                                                  -> read-only dataset browser confined to NVIZ_DATASETS_DIR (viz/datasets.py)
  GET /                                           -> a single static page that plots a tag of a run

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
    m = self._merged(run, "tag = ?", (tag,), rank)
    pts = sorted((step, v) for (_, step), (_, v) in m.items())
    return lttb(pts, points)

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
    return {"run": run, "ranks": len(files), "last_step": last_step, "last_ts_ms": last_ts}


def group_gpu(latest: Dict[str, Tuple[int, float]]) -> Dict[str, Dict[str, float]]:
  out: Dict[str, Dict[str, float]] = {}
  for tag, (_, v) in latest.items():
    m = re.fullmatch(r"gpu/(\d+)/(.+)", tag)
    if m:
      out.setdefault(m.group(1), {})[m.group(2)] = v
  return out


def group_router(latest: Dict[str, Tuple[int, float]]) -> Dict[str, Dict[str, float]]:
  out: Dict[str, Dict[str, float]] = {}
  for tag, (_, v) in latest.items():
    m = re.fullmatch(r"router/layer_(\d+)/(.+)", tag)
    if m:
      out.setdefault(f"layer_{m.group(1)}", {})[m.group(2)] = v
    elif tag.startswith("router_agg/"):
      out.setdefault("agg", {})[tag.split("/", 1)[1]] = v
  return out


def experiments(db_path: Optional[str]) -> List[dict]:
  if not db_path or not Path(db_path).exists():
    return []
  con = sqlite3.connect(f"file:{db_path}?mode=ro", uri=True, timeout=5.0)
  con.row_factory = sqlite3.Row
  try:
    exps = [dict(r) for r in con.execute("SELECT * FROM experiments ORDER BY created_at DESC")]
    for e in exps:
      runs = [dict(r) for r in con.execute("SELECT * FROM runs WHERE experiment_id = ? ORDER BY started_at DESC", (e["id"],))]
      for r in runs:
        for k in ("config_json", "results_json"):
          if r.get(k):
            try:
              r[k[:-5]] = json.loads(r.pop(k))
            except ValueError:
              pass
      e["runs"] = runs
    return exps
  except sqlite3.Error:
    return []
  finally:
    con.close()


_PAGE = """<!doctype html><meta charset=utf-8><title>nmoe_b200 runs</title>
<style>body{font:14px system-ui;margin:2em;max-width:1100px}select,input{font:inherit;margin-right:1em}canvas{border:1px solid #ccc;width:100%;height:420px}</style>
<h2>Training runs</h2><div><select id=run></select><input id=tag value="train/loss" size=32><button onclick=draw()>plot</button></div>
<canvas id=c width=1100 height=420></canvas><pre id=sum></pre>
<script>
async function j(u){return (await fetch(u)).json()}
async function init(){const r=await j('/api/runs');run.innerHTML=r.map(x=>`<option>${x.run}</option>`).join('');draw()}
async function draw(){if(!run.value)return;const s=await j(`/api/series?run=${run.value}&tag=${encodeURIComponent(tag.value)}&points=800`);
const p=s.points,g=c.getContext('2d');g.clearRect(0,0,c.width,c.height);if(!p.length)return;
const xs=p.map(a=>a[0]),ys=p.map(a=>a[1]),x0=Math.min(...xs),x1=Math.max(...xs),y0=Math.min(...ys),y1=Math.max(...ys);
g.beginPath();p.forEach((a,i)=>{const x=20+(a[0]-x0)/(x1-x0||1)*(c.width-40),y=c.height-20-(a[1]-y0)/(y1-y0||1)*(c.height-40);i?g.lineTo(x,y):g.moveTo(x,y)});g.stroke();
g.fillText(`${tag.value}: ${y0.toPrecision(4)} .. ${y1.toPrecision(4)}  steps ${x0}..${x1}`,24,14);
sum.textContent=JSON.stringify(await j(`/api/summary?run=${run.value}`),null,1)}
init()</script>"""


def make_handler(store: MetricStore, exp_db: Optional[str]):
  class Handler(BaseHTTPRequestHandler):
    def log_message(self, fmt, *args):   # quiet
      pass

    def _send(self, code: int, body, ctype: str = "application/json") -> None:
      data = body.encode() if isinstance(body, str) else json.dumps(body).encode()
      self.send_response(code)
      self.send_header("Content-Type", ctype)
      self.send_header("Content-Length", str(len(data)))
      self.end_headers()
      self.wfile.write(data)

    def _datasets(self, what: str, q: Dict[str, str]):
      """Read-only dataset browser (viz/datasets.py); every path is confined to NVIZ_DATASETS_DIR."""
      from . import datasets as D
      path = q.get("path", "")
      try:
        if what == "":
          return self._send(200, D.list_dir(path))
        if what == "preview":
          return self._send(200, D.preview_file(path, int(q.get("bytes", str(64 * 1024)))))
        if what == "meta":
          return self._send(200, D.meta(path))
        if what == "manifest":
          return self._send(200, D.manifest_preview(path, int(q.get("limit", "200"))))
        if what == "shard/stats":
          return self._send(200, D.shard_stats(path))
        if what == "shard/window":
          return self._send(200, D.token_window(path, int(q.get("offset", "0")), int(q.get("length", "256")),
                                                q.get("tokenizer")))
        if what == "index/header":
          return self._send(200, D.index_header(path))
        if what == "index/doc":
          return self._send(200, D.index_doc(path, int(q.get("doc", "0")), q.get("tokenizer")))
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
        if u.path == "/":
          return self._send(200, _PAGE, "text/html; charset=utf-8")
        if u.path == "/api/health":
          return self._send(200, {"ok": True, "runs": len(store.runs())})
        if u.path == "/api/runs":
          return self._send(200, [store.run_info(r) for r in store.runs()])
        if u.path == "/api/experiments":
          return self._send(200, experiments(exp_db))
        if u.path == "/api/datasets" or u.path.startswith("/api/datasets/"):
          return self._datasets(u.path[len("/api/datasets"):].strip("/"), q)
        run = q.get("run", "")
        if u.path.startswith("/api/") and run not in store.runs():
          return self._send(404, {"error": f"unknown run {run!r}"})
        if u.path == "/api/series":
          if "tag" not in q:
            return self._send(400, {"error": "tag is required"})
          n = max(3, min(int(q.get("points", "1000")), 5000))
          rank = int(q["rank"]) if "rank" in q else None
          pts = store.series(run, q["tag"], n, rank)
          return self._send(200, {"run": run, "tag": q["tag"], "points": [[s, v] for s, v in pts]})
        if u.path == "/api/summary":
          lat = store.latest(run, "%")
          keep = {t: {"step": s, "value": v} for t, (s, v) in sorted(lat.items())
                  if not t.startswith(("time_ms/", "gpu/", "router/layer_"))}
          return self._send(200, {"run": run, "latest": keep})
        if u.path == "/api/gpu":
          return self._send(200, {"run": run, "gpus": group_gpu(store.latest(run, "gpu/%"))})
        if u.path == "/api/router":
          lat = store.latest(run, "router%")
          return self._send(200, {"run": run, "router": group_router(lat)})
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
