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
