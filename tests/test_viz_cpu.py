"""Dashboard service: merged rank files, LTTB down-sampling, endpoint contract."""
import json
import threading
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
    runs = _get(port, "/api/runs")
    assert runs[0]["run"] == "runA" and runs[0]["ranks"] == 2 and runs[0]["last_step"] == 299
    s = _get(port, "/api/series?run=runA&tag=train/loss&points=50")
    assert len(s["points"]) == 50 and s["points"][0] == [0, 10.0]
    summ = _get(port, "/api/summary?run=runA")["latest"]
    assert "train/loss" in summ and not any(k.startswith("time_ms/") for k in summ)
    gpus = _get(port, "/api/gpu?run=runA")["gpus"]
    assert set(gpus) == {"0", "1"} and gpus["1"]["power_w"] == 710.0
    router = _get(port, "/api/router?run=runA")["router"]
    assert router["layer_01"]["cv"] == 0.1 and router["agg"]["mean_cv"] == 0.2
    assert _get(port, "/api/experiments") == []
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
