"""Dashboard service: merged rank files, LTTB down-sampling, endpoint contract."""
import json
import threading
import urllib.error
import urllib.request

from nmoe_b200.metrics import MetricsWriter
from nmoe_b200.viz.server import MetricStore, lttb, serve


def _get(port, path):
  with urllib.request.urlopen(f"http://127.0.0.1:{port}{path}", timeout=5) as r:
    return json.loads(r.read())


def test_lttb_keeps_ends_and_caps_points():
  pts = [(i, float((i * 37) % 101)) for i in range(5000)]
  out = lttb(pts, 200)
  assert len(out) == 200 and out[0] == pts[0] and out[-1] == pts[-1]
  assert [p[0] for p in out] == sorted(p[0] for p in out)
  assert lttb(pts[:50], 200) == pts[:50]


def test_endpoints_over_two_rank_files(tmp_path):
  w0 = MetricsWriter("runA", str(tmp_path), 0)
  w1 = MetricsWriter("runA", str(tmp_path), 1)
  for s in range(300):
    w0.insert_many(s, [("train/loss", 10.0 - s * 0.01), ("gpu/0/power_w", 700 + s % 5), ("router/layer_01/cv", 0.1),
                       ("router_agg/mean_cv", 0.2), ("time_ms/r0/step", 500.0)])
    w1.insert_many(s, [("gpu/1/power_w", 710.0), ("time_ms/r1/step", 501.0)])
  w0.close(); w1.close()
  store = MetricStore(str(tmp_path))
  assert store.runs() == ["runA"]
  assert len(store.series("runA", "train/loss", 100)) == 100
  srv = serve(str(tmp_path), None, port=0)
  port = srv.server_address[1]
  t = threading.Thread(target=srv.serve_forever, daemon=True)
  t.start()
  try:
    assert _get(port, "/api/health")["ok"]
    runs = _get(port, "/api/runs")["runs"]
    assert runs[0]["run"] == "runA" and runs[0]["ranks"] == 2 and runs[0]["last_step"] == 299 and runs[0]["last_ts"] > 0
    s = _get(port, "/api/series?run=runA&tag=train/loss&points=50")
    assert len(s["series"]) == 50 and s["series"][0]["step"] == 0 and s["series"][0]["value"] == 10.0 and s["series"][0]["ts_ms"] > 0
    tags = _get(port, "/api/tags?run=runA")["tags"]
    assert "train/loss" in tags and "gpu/1/power_w" in tags
    summ = _get(port, "/api/summary?run=runA")
    assert summ["summary"]["train/loss"] == 10.0 - 299 * 0.01 and summ["steps"]["train/loss"] == 299
    assert not any(k.startswith(("time_ms/", "gpu/")) for k in summ["summary"])
    g = _get(port, "/api/gpu?run=runA")
    assert [x["index"] for x in g["gpus"]] == [0, 1] and g["gpus"][1]["power_w"] == 710.0 and g["agg"] == {}
    router = _get(port, "/api/router?run=runA")
    assert router["layers"] == [{"idx": 1, "cv": 0.1}] and router["agg"] == {"router_agg/mean_cv": 0.2}
    assert _get(port, "/api/experiments") == {"experiments": []}
    assert _get(port, "/api/experiments/runs") == {"runs": []}
    for path, code in (("/api/series?run=runA", 400), ("/api/summary", 400), ("/api/summary?run=nope", 404), ("/api/experiments/run?run=runA", 404)):
      try:
        _get(port, path)
        raise AssertionError(path)
      except urllib.error.HTTPError as e:
        assert e.code == code, (path, e.code)
  finally:
    srv.shutdown()
    srv.server_close()


def test_dataset_browser_routes(tmp_path, monkeypatch):
  """/api/datasets/*: listing, shard statistics, token window, index header / document, manifest, flow directory,
  and refusal of paths that leave the datasets directory."""
  import urllib.error
  import numpy as np
  from nmoe_b200.data.sinks import ShardedWriter
  root = tmp_path / "data"
  src = root / "flows" / "dev" / "web"
  w = ShardedWriter(src, "web", "v1", num_shards=2, tokenizer="bytes", vocab_size=300, eos_token_id=256)
  rng = np.random.default_rng(0)
  for i in range(40):
    w.add_document(i % 2, rng.integers(0, 255, size=20 + i).tolist())
  w.finalize()
  (tmp_path / "secret.txt").write_text("outside")
  monkeypatch.setenv("NVIZ_DATASETS_DIR", str(root))
  srv = serve(str(tmp_path / "metrics"), None, port=0)
  port = srv.server_address[1]
  threading.Thread(target=srv.serve_forever, daemon=True).start()
  try:
    top = _get(port, "/api/datasets?path=flows/dev")
    assert [e["name"] for e in top["entries"]] == ["web"] and top["entries"][0]["kind"] == "dir"
    man = _get(port, "/api/datasets/manifest?path=flows/dev/web&limit=1")
    assert man["manifest"]["dataset"] == "web" and len(man["shards"]) == 1 and man["manifest"]["num_shards_listed"] == 2
    shard = "flows/dev/web/" + man["shards"][0]["path"]
    assert _get(port, f"/api/datasets/meta?path={shard}") | {} == _get(port, f"/api/datasets/meta?path={shard}")
    assert _get(port, f"/api/datasets/meta?path={shard}")["kind"] == "token_shard"
    st = _get(port, f"/api/datasets/shard/stats?path={shard}")
    assert st["documents"] == 20 and st["tokens"] == man["shards"][0]["num_tokens"] and st["max_token_id"] == 256
    win = _get(port, f"/api/datasets/shard/window?path={shard}&offset=3&length=5")
    assert len(win["ids"]) == 5 and win["start"] == 3
    idx = shard[:-4] + ".idx"
    hdr = _get(port, f"/api/datasets/index/header?path={idx}")
    assert hdr["documents"] == 20 and hdr["tokens_covered"] == st["tokens"]
    # the reference's parameter names for the same routes
    assert _get(port, f"/api/datasets/index/doc?shard_path={shard}&doc_idx=1&max_tokens=4")["ids"] == \
        _get(port, f"/api/datasets/index/doc?path={idx}&doc=1")["ids"][:4]
    assert len(_get(port, "/api/datasets/manifest?path=flows/dev/web&limit_shards=2")["shards"]) == 2
    (root / "notes.txt").write_text("line of text\n" * 500)
    assert _get(port, "/api/datasets/preview?path=notes.txt&max_bytes=2000")["bytes"] == 2000
    assert _get(port, "/api/datasets/preview?path=notes.txt&max_bytes=10")["bytes"] == 1024          # the floor
    doc = _get(port, f"/api/datasets/index/doc?path={idx}&doc=1")
    assert doc["tokens"] == len(doc["ids"]) and doc["ids"][-1] == 256
    flow = _get(port, "/api/datasets/pipeline?path=flows/dev")
    assert flow["sources"][0]["source"] == "web" and flow["total_tokens"] == man["manifest"]["total_tokens"]
    pv = _get(port, "/api/datasets/preview?path=flows/dev/web/manifest.json&bytes=2048")
    assert '"dataset"' in pv["text"]
    for bad in ("/api/datasets?path=../", "/api/datasets/preview?path=../secret.txt"):
      try:
        _get(port, bad)
        raise AssertionError("path traversal was served")
      except urllib.error.HTTPError as e:
        assert e.code == 400
  finally:
    srv.shutdown()


def test_runs_merge_with_the_experiments_database_and_its_routes(tmp_path):
  """The reference dashboard's contract (nviz/tests/api.runs.contract.test.ts, api.experiments.contract.test.ts): a run
  with metric files takes its status from the experiments database; a run known only to the database is listed with
  last_step 0 and last_ts 0; experiment summaries count runs by status."""
  import types
  from nmoe_b200.experiments import ExperimentTracker
  w = MetricsWriter("runA", str(tmp_path / "metrics"), 0)
  w.insert_many(1, [("train/loss", 10.0)])
  w.insert_many(2, [("train/loss", 8.0)])
  w.close()
  db = tmp_path / "experiments.db"
  cfg = types.SimpleNamespace(experiment_id="exp1", experiments_db=str(db), lr=0.1)
  tr = ExperimentTracker(cfg)
  assert tr.start_run("runA") == "runA" and tr.start_run("runB") == "runB" and tr.start_run("runC") == "runC"
  tr.update_results("runA", {"eval_loss": 3.5})
  tr.end_run("runB", "completed", {"final_loss": 2.5, "steps_completed": 7})
  tr.end_run("runC", "failed")
  assert tr.get_run("runB").status == "completed" and tr.get_run("runB")["ended_at"] and tr.get_run("nope") is None
  assert [r.id for r in tr.list_runs("exp1", status="running")] == ["runA"] and len(tr.list_runs("exp1")) == 3
  assert tr.get_experiment("exp1").project == "default" and [e.id for e in tr.list_experiments()] == ["exp1"]
  tr.start_run("runC")                                   # a resumed job re-opens its row
  assert tr.get_run("runC").status == "running" and tr.get_run("runC").ended_at is None
  tr.end_run("runC", "killed")
  made = tr.create_experiment("sweep", "moe", "lr sweep")
  assert made.startswith("moe_sweep_") and tr.get_experiment(made).description == "lr sweep"
  tr.close()
  srv = serve(str(tmp_path / "metrics"), str(db), port=0)
  port = srv.server_address[1]
  threading.Thread(target=srv.serve_forever, daemon=True).start()
  try:
    runs = {r["run"]: r for r in _get(port, "/api/runs")["runs"]}
    assert runs["runA"]["status"] == "running" and runs["runA"]["last_step"] == 2 and runs["runA"]["experiment_id"] == "exp1"
    assert runs["runB"]["status"] == "completed" and runs["runB"]["last_step"] == 0 and runs["runB"]["last_ts"] == 0
    assert list(runs)[0] == "runA"                       # newest metric activity first
    exps = {e["id"]: e for e in _get(port, "/api/experiments")["experiments"]}
    e = exps["exp1"]
    assert (e["runs_total"], e["runs_running"], e["runs_completed"], e["runs_failed"], e["runs_killed"]) == (3, 1, 1, 0, 1)
    assert e["name"] == "exp1" and e["project"] == "default" and e["last_started_at"] and exps[made]["runs_total"] == 0
    rows = _get(port, "/api/experiments/runs?experiment_id=exp1&limit=2")["runs"]
    assert len(rows) == 2 and {"run", "experiment_id", "status", "started_at", "ended_at", "git_hash", "git_dirty", "config_json",
                               "results_json", "last_ts", "last_step"} <= set(rows[0])
    one = _get(port, "/api/experiments/run?run=runB")["run"]
    assert one["status"] == "completed" and json.loads(one["results_json"])["steps_completed"] == 7 and json.loads(one["config_json"])["lr"] == 0.1
  finally:
    srv.shutdown()
    srv.server_close()


def test_experiments_database_of_the_earlier_layout_is_upgraded(tmp_path):
  import sqlite3
  import types
  from nmoe_b200.experiments import ExperimentTracker
  db = tmp_path / "old.db"
  con = sqlite3.connect(db)
  con.executescript(
    "CREATE TABLE experiments (id TEXT PRIMARY KEY, created_at REAL, description TEXT);"
    "CREATE TABLE runs (id TEXT PRIMARY KEY, experiment_id TEXT, config_json TEXT, git_hash TEXT, git_dirty INTEGER,"
    " started_at REAL, ended_at REAL, status TEXT, results_json TEXT);"
    "INSERT INTO experiments VALUES ('old', 1700000000.0, '');"
    "INSERT INTO runs VALUES ('r0', 'old', '{}', 'abc', 0, 1700000000.0, 1700003600.0, 'completed', NULL);")
  con.commit(); con.close()
  tr = ExperimentTracker(types.SimpleNamespace(experiment_id="old", experiments_db=str(db)))
  assert tr.get_experiment("old").name == "old" and tr.get_experiment("old").created_at == "2023-11-14 22:13:20"
  r = tr.get_run("r0")
  assert r.started_at == "2023-11-14 22:13:20" and r.ended_at == "2023-11-14 23:13:20"
  tr.start_run("r1")
  assert [x.id for x in tr.list_runs("old")] == ["r1", "r0"]
  tr.close()


def _js_balance(src):
  """A structural check of a script without a JavaScript engine: strings, template literals (with ${} nesting),
  comments and regex literals are skipped; every bracket must close in order."""
  stack, i, n, prev = [], 0, len(src), ""
  pairs = {")": "(", "]": "[", "}": "{"}
  while i < n:
    c = src[i]
    if c in " \t\r\n":
      i += 1
      continue
    if src.startswith("//", i):
      i = src.index("\n", i) if "\n" in src[i:] else n
      continue
    if src.startswith("/*", i):
      i = src.index("*/", i) + 2
      continue
    if c in "'\"":
      j = i + 1
      while src[j] != c:
        assert src[j] != "\n", f"string runs over a line end at offset {i}"
        j += 2 if src[j] == "\\" else 1
      i, prev = j + 1, "s"
      continue
    if c == "`":
      stack.append("`")
      i += 1
      # template text up to the closing back-tick or a ${ that opens an expression
      while True:
        if src[i] == "\\":
          i += 2
        elif src[i] == "`":
          assert stack.pop() == "`"
          i += 1
          break
        elif src.startswith("${", i):
          stack.append("${")
          i += 2
          break
        else:
          i += 1
      prev = "s"
      continue
    if c == "/" and prev in "(,=:[!&|?{};\n" + "":
      j = i + 1
      in_class = False
      while src[j] != "/" or in_class:
        in_class = (src[j] == "[") or (in_class and src[j] != "]")
        j += 2 if src[j] == "\\" else 1
      i, prev = j + 1, "s"
      continue
    if c in "([{":
      stack.append(c)
    elif c in ")]":
      assert stack and stack.pop() == pairs[c], f"unbalanced {c} at offset {i}: ...{src[max(0, i - 60):i + 1]}"
    elif c == "}":
      assert stack, f"unbalanced }} at offset {i}"
      top = stack.pop()
      if top == "${":                      # back inside the template text
        while True:
          if src[i + 1] == "\\":
            i += 2
          elif src[i + 1] == "`":
            assert stack.pop() == "`"
            i += 1
            break
          elif src.startswith("${", i + 1):
            stack.append("${")
            i += 2
            break
          else:
            i += 1
      else:
        assert top == "{", f"unbalanced }} at offset {i}: ...{src[max(0, i - 60):i + 1]}"
    prev = c
    i += 1
  assert not stack, f"unclosed {stack[-3:]}"


def test_dashboard_page_is_served_and_its_scripts_are_well_formed(tmp_path):
  from nmoe_b200.viz.server import STATIC_DIR, static_file
  srv = serve(str(tmp_path), None, port=0)
  port = srv.server_address[1]
  threading.Thread(target=srv.serve_forever, daemon=True).start()
  try:
    with urllib.request.urlopen(f"http://127.0.0.1:{port}/", timeout=5) as r:
      page = r.read().decode()
      assert r.headers["Content-Type"].startswith("text/html")
    import re
    scripts = re.findall(r'<script src="/static/([\w.]+)"', page)
    assert scripts == ["chart.js", "app.js", "panels.js"] and 'href="/static/style.css"' in page
    ids_in_page = set(re.findall(r'id="([\w-]+)"', page))
    for name in scripts:
      with urllib.request.urlopen(f"http://127.0.0.1:{port}/static/{name}", timeout=5) as r:
        src = r.read().decode()
        assert "javascript" in r.headers["Content-Type"]
      _js_balance(src)
      for ref in re.findall(r"\$\('([\w-]+)'\)", src):        # every element the scripts look up exists
        assert ref in ids_in_page or ref in ("open-run", "ds-off", "ds-win", "ds-doc", "ds-docbtn", "ds-tokens", "ds-docout"), ref
      for url in re.findall(r"['`](/api/[\w/]+)", src):          # every route the scripts call is one the server has
        assert url.rstrip("/") in {"/api/runs", "/api/series", "/api/summary", "/api/tags", "/api/gpu", "/api/router", "/api/experiments",
                       "/api/experiments/runs", "/api/datasets", "/api/datasets/manifest", "/api/datasets/pipeline",
                       "/api/datasets/meta", "/api/datasets/shard/stats", "/api/datasets/shard/window",
                       "/api/datasets/index/doc", "/api/datasets/index/header", "/api/datasets/preview"}, url
    for bad in ("/static/../server.py", "/static/nope.js", "/static/%2e%2e/server.py"):
      try:
        urllib.request.urlopen(f"http://127.0.0.1:{port}{bad}", timeout=5)
        raise AssertionError(bad)
      except urllib.error.HTTPError as e:
        assert e.code == 404
    assert static_file("../server.py") is None and STATIC_DIR.name == "static"
  finally:
    srv.shutdown()
    srv.server_close()


def test_gpu_telemetry_rows_use_the_dashboard_tag_names():
  from nmoe_b200.utils.gpu_telemetry import _FIELDS, dashboard_items
  snap = [dict(zip(_FIELDS, (0, 97, 40, 150 << 30, 180 << 30, 812000, 71, 1560, 1965, 0x4, 0, 123))),
          dict(zip(_FIELDS, (1, 91, 38, 148 << 30, 180 << 30, 640000, 78, 1900, 1965, 0x20 | 0x8, 2, 123)))]
  rows = dict(dashboard_items(snap))
  assert rows["gpu/0/utilization_gpu"] == 97.0 and rows["gpu/0/memory_used_gib"] == 150.0 and rows["gpu/0/power_draw_w"] == 812.0
  assert rows["gpu/0/throttle_power"] == 1.0 and rows["gpu/0/throttle_thermal"] == 0.0 and rows["gpu/0/throttle_hw_slowdown"] == 0.0
  assert rows["gpu/1/throttle_thermal"] == 1.0 and rows["gpu/1/throttle_hw_slowdown"] == 1.0 and rows["gpu/1/ecc_uncorrected"] == 2.0
  assert rows["gpu/1/clocks_sm_mhz"] == 1900.0 and rows["gpu/1/clocks_sm_max_mhz"] == 1965.0
  assert rows["gpu_agg/mean_utilization_gpu"] == 94.0 and rows["gpu_agg/total_memory_used_gib"] == 298.0
  assert rows["gpu_agg/total_power_w"] == 1452.0 and rows["gpu_agg/max_temperature_c"] == 78.0
  assert dashboard_items([]) == []


def test_html_report_is_self_contained_and_compares_runs(tmp_path):
  import re
  import types
  import xml.etree.ElementTree as ET
  from nmoe_b200.experiments import ExperimentTracker
  from nmoe_b200.viz.report import build_report, main, svg_chart
  for run, slope in (("base", 0.01), ("trial", 0.02)):
    w = MetricsWriter(run, str(tmp_path / "m"), 0)
    for s in range(1, 121):
      w.insert_many(s, [("train/loss", 10.0 - slope * s), ("optimizer/lr", 1e-3 * min(1.0, s / 20)), ("router/layer_01/cv", 0.2),
                        ("router/layer_01/entropy", 1.9), ("router_agg/mean_cv", 0.2), ("eval/task/arc/acc", 0.4), ("eval/task/arc/centered", 0.2),
                        ("eval/task/arc/n", 100.0), ("eval/CORE", 0.2)])
    w.close()
  db = tmp_path / "e.db"
  tr = ExperimentTracker(types.SimpleNamespace(experiment_id="exp", experiments_db=str(db), lr=0.5))
  tr.start_run("trial"); tr.end_run("trial", "completed", {"final_loss": 7.6}); tr.close()
  out = tmp_path / "r.html"
  assert main(["--metrics-dir", str(tmp_path / "m"), "--run", "trial", "--compare", "base", "--experiments-db", str(db), "--output", str(out)]) == 0
  page = out.read_text()
  assert "<script" not in page and "http://" not in page.replace("http://www.w3.org/2000/svg", "") and "https://" not in page
  assert "status completed" in page and "final_loss" in page and "compared with" in page and "CORE = 0.2000" in page
  svgs = re.findall(r"<svg.*?</svg>", page, flags=re.S)
  assert len(svgs) >= 4
  for s in svgs:
    ET.fromstring(s)                                              # every chart is well-formed XML
  loss = next(s for s in svgs if s.count("<polyline") == 2)       # two runs overlaid
  assert loss.count("<polyline") == 2
  assert "no data" in svg_chart([("x", [])]) and "<circle" in svg_chart([("x", [(1, 2.0)])])
  assert "<polyline" in svg_chart([("x", [(1, 1e-4), (2, 1e-2), (3, 0.0)])], log_y=True)          # the zero is left out on a log axis
  import pytest
  with pytest.raises(KeyError):
    build_report(MetricStore(str(tmp_path / "m")), "nope")
  assert main(["--metrics-dir", str(tmp_path / "m"), "--run", "nope", "--output", str(out)]) == 1


def test_dashboard_image_file_list_covers_the_servers_imports(tmp_path):
  """docker/Dockerfile.viz copies a hand-picked set of modules: run the server's imports and one dataset route in a
  tree that holds exactly those files, so a new import cannot silently break the slim image."""
  import re
  import shutil
  import subprocess
  import sys
  from pathlib import Path
  root = Path(__file__).resolve().parent.parent
  text = (root / "docker" / "Dockerfile.viz").read_text().replace("\\\n", " ")
  stage = tmp_path / "workspace"
  for line in text.splitlines():
    if line.startswith("COPY "):
      *srcs, dst = line.split()[1:]
      for s in srcs:
        target = stage / dst.replace("/workspace/", "")
        if (root / s).is_dir():
          shutil.copytree(root / s, target, ignore=shutil.ignore_patterns("__pycache__"))
        else:
          dest = target / Path(s).name if dst.endswith("/") else target
          dest.parent.mkdir(parents=True, exist_ok=True)
          shutil.copy(root / s, dest)
  data = tmp_path / "data"
  data.mkdir()
  import numpy as np
  np.save(data / "s.npy", np.arange(10, dtype=np.uint32))
  code = ("import nmoe_b200.viz.server as S, nmoe_b200.viz.report, nmoe_b200.viz.datasets as D; "
          "print(D.shard_stats('s.npy')['tokens'], S.static_file('index.html') is not None)")
  out = subprocess.run([sys.executable, "-c", code], cwd=stage, capture_output=True, text=True,
                       env={"PATH": "/usr/bin:/bin", "PYTHONPATH": str(stage), "NVIZ_DATASETS_DIR": str(data)})
  assert out.returncode == 0 and out.stdout.split() == ["10", "True"], out.stderr[-2000:]


def test_server_answers_malformed_requests_without_dying(tmp_path):
  """Bad numbers, unknown routes, odd paths: an error body and the right status, and the next request still works."""
  w = MetricsWriter("r", str(tmp_path), 0)
  w.insert_many(1, [("train/loss", 1.0)])
  w.close()
  srv = serve(str(tmp_path), None, port=0)
  port = srv.server_address[1]
  threading.Thread(target=srv.serve_forever, daemon=True).start()
  try:
    for path, code in (("/api/series?run=r&tag=train/loss&points=abc", 400), ("/api/series?run=r&tag=train/loss&rank=x", 400),
                       ("/api/nope?run=r", 404), ("/api/experiments/runs?limit=many", 400), ("/api/experiments/run", 400),
                       ("/api/datasets/shard/window?path=x&offset=-1&length=zz", 400), ("/static/", 200), ("/api/runs?x=%ff%fe", 200),
                       ("/api/series?run=../../etc&tag=t", 404), ("/api/tags?run=r%00", 404)):
      try:
        with urllib.request.urlopen(f"http://127.0.0.1:{port}{path}", timeout=5) as r:
          got = r.status
      except urllib.error.HTTPError as e:
        got = e.code
        json.loads(e.read())                                # errors are JSON too
      assert got == code, (path, got)
    assert _get(port, "/api/series?run=r&tag=train/loss")["series"][0]["value"] == 1.0
    assert _get(port, "/api/series?run=r&tag=no/such/tag")["series"] == []
  finally:
    srv.shutdown()
    srv.server_close()
