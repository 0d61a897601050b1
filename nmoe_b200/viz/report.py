"""A run as one self-contained HTML file: summary, charts (inline SVG), router table, evaluation results.

  python -m nmoe_b200.viz.report --metrics-dir /data/metrics --run RUN [--compare OTHER ...] --output run.html

For clusters where no port can be opened for the dashboard, and for attaching a run to a ticket or a merge request:
the file has no scripts and no external references, so it opens anywhere and stays readable in an archive.  It reads
the same per-rank metric files as the dashboard (``viz.server.MetricStore``) and, when given, the experiments database.
"""
from __future__ import annotations

import argparse
import html
import json
import time
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

from .server import ExperimentsView, MetricStore, group_router

COLORS = ("#2563eb", "#ea580c", "#16a34a", "#dc2626", "#7c3aed", "#0891b2")
DEFAULT_TAGS = ("train/loss", "optimizer/lr", "throughput/tokens_per_s_gpu", "throughput/ms_per_step", "efficiency/tflops",
                "train/grad_norm", "memory/max_alloc_gib", "router_agg/mean_cv", "router_agg/max_load", "eval/CORE")


def _fmt(v: Optional[float]) -> str:
  if v is None:
    return "–"
  a = abs(v)
  if a == 0:
    return "0"
  if a >= 1e6:
    return f"{v:,.0f}"
  if a >= 100:
    return f"{v:.1f}"
  if a >= 1:
    return f"{v:.4g}"
  return f"{v:.3e}" if a < 1e-3 else f"{v:.4f}"


def svg_chart(series: Sequence[Tuple[str, List[Tuple[int, float]]]], width: int = 560, height: int = 220, log_y: bool = False) -> str:
  """Line chart of several (name, [(step, value)]) series as an SVG string; empty series are skipped."""
  import math
  ml, mr, mt, mb = 56, 10, 10, 24
  pts = [(n, [(s, v) for s, v in p if math.isfinite(v) and (not log_y or v > 0)]) for n, p in series]
  pts = [(n, p) for n, p in pts if p]
  if not pts:
    return f'<svg width="{width}" height="{height}"><text x="{ml}" y="{height // 2}" fill="#888" font-size="12">no data</text></svg>'
  f = (lambda v: math.log10(v)) if log_y else (lambda v: v)
  xs = [s for _, p in pts for s, _ in p]
  ys = [f(v) for _, p in pts for _, v in p]
  x0, x1, y0, y1 = min(xs), max(xs), min(ys), max(ys)
  if x1 == x0:
    x1 = x0 + 1
  if y1 == y0:
    pad = abs(y0) * 0.05 or 1.0
    y0, y1 = y0 - pad, y1 + pad
  X = lambda s: ml + (s - x0) / (x1 - x0) * (width - ml - mr)
  Y = lambda v: height - mb - (f(v) - y0) / (y1 - y0) * (height - mt - mb)
  out = [f'<svg xmlns="http://www.w3.org/2000/svg" width="{width}" height="{height}" font-family="system-ui, sans-serif" font-size="11">']
  for k in range(5):
    yy = y0 + (y1 - y0) * k / 4
    py = height - mb - (height - mt - mb) * k / 4
    out.append(f'<line x1="{ml}" y1="{py:.1f}" x2="{width - mr}" y2="{py:.1f}" stroke="#e5e7eb"/>')
    out.append(f'<text x="{ml - 4}" y="{py + 3:.1f}" text-anchor="end" fill="#6b7280">{_fmt(10 ** yy if log_y else yy)}</text>')
  for k in range(5):
    xx = x0 + (x1 - x0) * k / 4
    out.append(f'<text x="{X(xx):.1f}" y="{height - 6}" text-anchor="middle" fill="#6b7280">{int(round(xx))}</text>')
  for i, (name, p) in enumerate(pts):
    path = " ".join(f"{X(s):.1f},{Y(v):.1f}" for s, v in p)
    c = COLORS[i % len(COLORS)]
    if len(p) == 1:
      out.append(f'<circle cx="{X(p[0][0]):.1f}" cy="{Y(p[0][1]):.1f}" r="3" fill="{c}"/>')
    else:
      out.append(f'<polyline fill="none" stroke="{c}" stroke-width="1.5" points="{path}"/>')
  out.append("</svg>")
  return "".join(out)


def _table(headers: Iterable[str], rows: Iterable[Iterable]) -> str:
  head = "".join(f"<th>{html.escape(str(h))}</th>" for h in headers)
  body = "".join("<tr>" + "".join(f"<td>{html.escape(str(c))}</td>" for c in r) + "</tr>" for r in rows)
  return f"<table><tr>{head}</tr>{body}</table>"


def build_report(store: MetricStore, run: str, compare: Sequence[str] = (), tags: Sequence[str] = DEFAULT_TAGS,
                 experiments_db: Optional[str] = None, points: int = 600) -> str:
  runs = [run] + [r for r in compare if r != run]
  known = set(store.runs())
  missing = [r for r in runs if r not in known]
  if missing:
    raise KeyError(f"no metric files for run(s) {missing}; known runs: {sorted(known)}")
  info = store.run_info(run)
  latest = store.latest(run, "%")
  row = ExperimentsView(experiments_db).run(run) if experiments_db else None
  parts: List[str] = []
  parts.append(f"<h1>{html.escape(run)}</h1>")
  meta = [f"last step {info['last_step']}", f"{info['ranks']} rank file(s)",
          "last write " + time.strftime("%Y-%m-%d %H:%M:%S UTC", time.gmtime(info["last_ts"] / 1000)) if info["last_ts"] else "no timestamps"]
  if row:
    meta += [f"status {row['status']}", f"experiment {row['experiment_id']}", f"git {(row['git_hash'] or '')[:12]}{' (dirty)' if row['git_dirty'] else ''}",
             f"started {row['started_at']}"] + ([f"ended {row['ended_at']}"] if row["ended_at"] else [])
  parts.append('<p class="meta">' + " · ".join(html.escape(m) for m in meta) + "</p>")
  if len(runs) > 1:
    legend = " ".join(f'<span class="sw" style="background:{COLORS[i % len(COLORS)]}"></span>{html.escape(r)}' for i, r in enumerate(runs))
    parts.append(f'<p class="meta">compared with: {legend}</p>')

  # summary cards
  cards = []
  for tag in tags:
    if tag in latest:
      step, v = latest[tag]
      cards.append(f'<div class="card"><div class="k">{html.escape(tag)}</div><div class="v">{_fmt(v)}</div><div class="s">step {step}</div></div>')
  parts.append('<div class="cards">' + "".join(cards) + "</div>")

  # charts
  parts.append("<h2>Curves</h2><div class='charts'>")
  for tag in tags:
    series = [(r, store.series(r, tag, points)) for r in runs]
    if not any(p for _, p in series):
      continue
    log_y = tag == "optimizer/lr" and all(v > 0 for _, p in series for _, v in p)
    parts.append(f"<figure><figcaption>{html.escape(tag)}</figcaption>{svg_chart(series, log_y=log_y)}</figure>")
  parts.append("</div>")

  # router
  layers, agg = group_router({t: sv for t, sv in latest.items() if t.startswith("router")})
  if layers:
    keys = ("cv", "entropy", "max_load", "bias_range", "experts_active")
    parts.append("<h2>Router, latest step</h2>")
    parts.append(_table(("layer",) + keys, [[l["idx"]] + [_fmt(l.get(k)) for k in keys] for l in layers]))
    if agg:
      parts.append('<p class="meta">' + " · ".join(f"{html.escape(k)} = {_fmt(v)}" for k, v in sorted(agg.items())) + "</p>")

  # evaluation
  ev = {t: sv for t, sv in latest.items() if t.startswith("eval/task/")}
  if ev:
    tasks: Dict[str, Dict[str, float]] = {}
    for t, (_, v) in ev.items():
      _, _, name, key = t.split("/", 3)
      tasks.setdefault(name, {})[key] = v
    parts.append("<h2>Evaluation, latest</h2>")
    parts.append(_table(("task", "acc", "centred", "n"), [[n, _fmt(d.get("acc")), _fmt(d.get("centered")), int(d.get("n", 0))] for n, d in sorted(tasks.items())]))
    if "eval/CORE" in latest:
      parts.append(f'<p class="meta">CORE = {_fmt(latest["eval/CORE"][1])} at step {latest["eval/CORE"][0]}</p>')

  # configuration and results from the experiments database
  if row:
    for title, key in (("Results", "results_json"), ("Configuration", "config_json")):
      if row.get(key):
        try:
          text = json.dumps(json.loads(row[key]), indent=1, sort_keys=True)
        except ValueError:
          text = str(row[key])
        parts.append(f"<h2>{title}</h2><pre>{html.escape(text)}</pre>")

  css = ("body{font:14px/1.45 system-ui,sans-serif;margin:2em auto;max-width:1200px;padding:0 1em;color:#111}"
         "h1{margin-bottom:.2em}.meta{color:#6b7280}.cards{display:grid;grid-template-columns:repeat(auto-fill,minmax(190px,1fr));gap:8px}"
         ".card{border:1px solid #e5e7eb;border-radius:6px;padding:8px}.k{font-size:11px;color:#6b7280}.v{font-size:20px}.s{font-size:11px;color:#6b7280}"
         ".charts{display:grid;grid-template-columns:repeat(auto-fill,minmax(570px,1fr));gap:10px}figure{margin:0;border:1px solid #e5e7eb;border-radius:6px;padding:6px}"
         "figcaption{font-size:12px;font-weight:600}table{border-collapse:collapse}td,th{border-bottom:1px solid #e5e7eb;padding:3px 10px;text-align:right}"
         "th{color:#6b7280;font-weight:500}pre{background:#f9fafb;border:1px solid #e5e7eb;border-radius:6px;padding:8px;overflow:auto}"
         ".sw{display:inline-block;width:10px;height:10px;border-radius:2px;margin:0 4px 0 10px}")
  return (f"<!doctype html><html><head><meta charset='utf-8'><title>{html.escape(run)}</title><style>{css}</style></head><body>"
          + "".join(parts) + f"<p class='meta'>generated {time.strftime('%Y-%m-%d %H:%M:%S UTC', time.gmtime())}</p></body></html>")


def main(argv=None) -> int:
  ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
  ap.add_argument("--metrics-dir", required=True); ap.add_argument("--run", required=True); ap.add_argument("--output", required=True)
  ap.add_argument("--compare", action="append", default=[], help="another run to overlay on the charts; repeatable")
  ap.add_argument("--experiments-db"); ap.add_argument("--tag", action="append", help="chart this tag (repeatable) instead of the default set")
  ap.add_argument("--points", type=int, default=600)
  a = ap.parse_args(argv)
  try:
    text = build_report(MetricStore(a.metrics_dir), a.run, a.compare, tuple(a.tag) if a.tag else DEFAULT_TAGS, a.experiments_db, a.points)
  except KeyError as e:
    print(str(e.args[0]))
    return 1
  with open(a.output, "w", encoding="utf-8") as f:
    f.write(text)
  print(f"{a.output}: {len(text) / 1024:.0f} KiB")
  return 0


if __name__ == "__main__":
  raise SystemExit(main())
