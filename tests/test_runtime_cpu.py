"""Config precedence, fingerprint, WSD schedule, loader determinism/resume, checkpoint atomicity,
metrics store, experiments DB -- all on CPU."""
import json
import math
import os

import numpy as np
import pytest
import torch

from nmoe_b200 import config as C
from nmoe_b200.opt import scheduled_lrs, wsd_scale


def test_config_precedence_and_fingerprint(tmp_path):
  p = tmp_path / "c.toml"
  p.write_text('dim = 64\nn_layers = 2\nn_heads = 2\nsteps = 10\nbatch_size = 4\ndtype = "bf16"\n[attn_swa]\nkv_heads = 1\n')
  cfg = C.from_toml(p, ["--steps=7", "--no-resume", "--lr_dense", "1e-3"], env={"NMOE_STEPS": "5", "NMOE_BATCH_SIZE": "8"})
  assert cfg.steps == 7 and cfg.batch_size == 8 and cfg.resume is False and cfg.lr_dense == 1e-3
  assert cfg.attn_swa == {"kv_heads": 1}
  fp1 = C.fingerprint(cfg)
  cfg.steps = 8
  assert C.fingerprint(cfg) != fp1 and len(fp1) == 64
  with pytest.raises(TypeError):
    C.from_toml(p, ["--no_such_key=1"])


def test_env_expansion_allowlist(tmp_path):
  p = tmp_path / "m.toml"
  p.write_text('a = "${NMOE_X:-dflt}/z"\nb = "${HOME}"\n')
  with pytest.raises(C.ConfigEnvError):
    C.load_toml(p)
  p.write_text('a = "${NMOE_X:-dflt}/z"\n')
  assert C.load_toml(p)["a"] == "dflt/z"
  os.environ["NMOE_X"] = "v"
  try:
    assert C.load_toml(p)["a"] == "v/z"
  finally:
    del os.environ["NMOE_X"]
  p.write_text('a = "${NMOE_UNSET_VAR}"\n')
  with pytest.raises(C.ConfigEnvError):
    C.load_toml(p)


def test_wsd_schedule():
  cfg = C.Config(dim=8, n_layers=1, n_heads=1, warmup_steps=10, hold_tokens=1000, decay_tokens=1000, decay_floor=1e-5,
                 lr_dense=1e-3, lr_expert=1e-2, lr_router=1e-6)
  assert wsd_scale(0, 0, cfg) == pytest.approx(0.1)
  assert wsd_scale(50, 500, cfg) == 1.0
  assert wsd_scale(50, 1500, cfg) == pytest.approx(0.5)
  assert wsd_scale(50, 5000, cfg) == 0.0
  lrs = scheduled_lrs(50, 5000, cfg)
  assert lrs["dense"] == pytest.approx(1e-5) and lrs["router"] == pytest.approx(1e-6)


def _make_shards(d, n_files=3, n_tok=1000):
  rng = np.random.default_rng(0)
  for i in range(n_files):
    np.save(d / f"s{i}.npy", rng.integers(0, 5000, size=n_tok + i * 17, dtype=np.uint32))


def test_loader_global_stream_is_world_invariant_and_resumes(tmp_path):
  from nmoe_b200.data.loader import build_loader
  _make_shards(tmp_path)
  cfg = C.Config(dim=8, n_layers=1, n_heads=1, data_path=str(tmp_path), batch_size=4, seq_len=16, steps=100)
  one, _ = build_loader(cfg, 0, 1, print_fn=lambda *a: None)
  two = [build_loader(cfg, r, 2, print_fn=lambda *a: None)[0] for r in range(2)]
  for _ in range(40):      # crosses file boundaries and wraps
    x1, y1 = one.next()
    xs = torch.cat([l.next()[0] for l in two])
    assert torch.equal(x1, xs)
    assert torch.equal(x1[:, 1:], y1[:, :-1])
  state = one.state_dict()
  nxt = one.next()[0]
  fresh, _ = build_loader(cfg, 0, 1, print_fn=lambda *a: None)
  fresh.load_state_dict(json.loads(json.dumps(state)))
  assert torch.equal(fresh.next()[0], nxt)
  assert state["cursors"]["data_path"]["wrap_count"] >= 0


def test_mixture_plan_quota_and_swrr(tmp_path):
  from nmoe_b200.data.mixture import largest_remainder_quota, resolve_plan
  assert sum(largest_remainder_quota(1000 * 16, 16, [1.0, 2.0, 3.0])) == 1000
  (tmp_path / "mix.toml").write_text(
    '[mixtures.m]\ntotal_tokens_b = 1.0\n[[mixtures.m.sources]]\nid = "a"\ntokens_b = 0.75\n'
    '[[mixtures.m.sources]]\nid = "b"\ntokens_b = 0.25\n')
  (tmp_path / "flow.toml").write_text('[flow.dev]\nmode = "dev"\ntokens_b = 0.000016\n[flow.dev.mixture]\npretrain = "m"\n')
  plan = resolve_plan(mixture_toml=tmp_path / "mix.toml", flow_profiles_toml=tmp_path / "flow.toml",
                      flow_section="flow.dev", seq_len=16)
  q = [s.quota_sequences for s in plan.stages[0].sources]
  assert sum(q) == 1000 and q == [750, 250] and len(plan.plan_hash) == 64
  plan2 = resolve_plan(mixture_toml=tmp_path / "mix.toml", flow_profiles_toml=tmp_path / "flow.toml",
                       flow_section="flow.dev", seq_len=32)
  assert plan2.plan_hash != plan.plan_hash


def _tiny_cfg(tmp_path, **kw):
  base = dict(vocab_size=256, eos_token_id=255, dim=64, n_layers=2, n_heads=2, inter_dim=128, moe_inter_dim=32,
              n_routed_experts=4, n_activated_experts=2, n_shared_experts=1, n_dense_layers=1, q_lora_rank=32,
              kv_lora_rank=16, qk_nope_head_dim=16, qk_rope_head_dim=8, v_head_dim=16, batch_size=2, seq_len=32,
              max_position_embeddings=64, warmup_steps=2, steps=6, log_every=2, checkpoint_every=3,
              checkpoint_dir=str(tmp_path / "ckpt"), metrics_dir=str(tmp_path / "metrics"),
              experiments_db=str(tmp_path / "exp.db"), data_path="synthetic", activation_checkpoint="none")
  base.update(kw)
  return C.Config(**base)


def test_train_checkpoint_resume_is_exact(tmp_path, monkeypatch):
  from nmoe_b200.train import train
  monkeypatch.setenv("NMOE_RUN", "t1")
  full = train(_tiny_cfg(tmp_path / "a"))
  # same run split in two: 3 steps, then resume to 6
  monkeypatch.setenv("NMOE_RUN", "t2")
  cfg_b = _tiny_cfg(tmp_path / "b")
  cfg_b3 = _tiny_cfg(tmp_path / "b", steps=3)
  # identical fingerprints are required for resume, so run the first half with steps=6 and stop via checkpoint
  import nmoe_b200.train as T
  real_save = T.__dict__.get("save_checkpoint")
  first = train(_tiny_cfg(tmp_path / "b", steps=6, checkpoint_every=3))
  assert first["final_loss"] == pytest.approx(full["final_loss"], abs=1e-6)
  # drop the final checkpoint so that the latest finalised step is 3, then resume
  import shutil
  from nmoe_b200.checkpoint import TRACKER, iteration_dir
  shutil.rmtree(iteration_dir(tmp_path / "b" / "ckpt", 6))
  (tmp_path / "b" / "ckpt" / TRACKER).write_text("3")
  resumed = train(cfg_b)
  assert resumed["final_loss"] == pytest.approx(full["final_loss"], abs=1e-6)
  assert resumed["tokens_seen"] == full["tokens_seen"]


def test_checkpoint_crash_between_files_keeps_previous_step(tmp_path):
  from nmoe_b200.checkpoint import Checkpointer, iteration_dir, read_tracker, try_finalize_step
  ck = Checkpointer(str(tmp_path), keep_last=2, async_io=False)
  for step in (1, 2):
    ck.submit(iteration_dir(tmp_path, step) / "rd.pt", {"step": step}, step, 2)
    ck.submit(iteration_dir(tmp_path, step) / "dp_rank_000.pt", {"step": step}, step, 2)
  assert read_tracker(tmp_path) == -1                     # rank 1's file never arrived
  ck.submit(iteration_dir(tmp_path, 1) / "dp_rank_001.pt", {"step": 1}, 1, 2)
  assert read_tracker(tmp_path) == 1 and ck.find_latest(0) == 1
  assert not (iteration_dir(tmp_path, 2) / "manifest.json").exists()
  # a writer that dies mid-write: error is latched and raised on the next call
  def boom(stage):
    if stage == "after_write":
      raise OSError("disk full")
  ck2 = Checkpointer(str(tmp_path), async_io=True, fault_hook=boom)
  ck2.submit(iteration_dir(tmp_path, 3) / "rd.pt", {"step": 3}, 3, 1)
  with pytest.raises(RuntimeError, match="disk full"):
    ck2.wait()
  ck2.close()
  assert read_tracker(tmp_path) == 1


def test_resume_refuses_other_config(tmp_path, monkeypatch):
  from nmoe_b200.train import train
  monkeypatch.setenv("NMOE_RUN", "t3")
  train(_tiny_cfg(tmp_path, steps=3))
  with pytest.raises(RuntimeError, match="fingerprint"):
    train(_tiny_cfg(tmp_path, steps=3, lr_dense=1e-3))


def test_metrics_store_and_experiments(tmp_path, monkeypatch):
  from nmoe_b200.train import train
  from nmoe_b200.metrics import MetricsWriter
  from nmoe_b200.experiments import ExperimentTracker
  monkeypatch.setenv("NMOE_RUN", "runX")
  cfg = _tiny_cfg(tmp_path)
  train(cfg)
  w = MetricsWriter("runX", cfg.metrics_dir, 0)
  loss = w.query("train/loss")
  assert [s for s, _ in loss] == [1, 2, 4, 6] and all(math.isfinite(v) for _, v in loss)
  assert w.query("router/layer_00/cv") and w.query("throughput/tokens_per_s_gpu")
  w.close()
  tr = ExperimentTracker(cfg)
  run = tr.get_run("runX")
  assert run["status"] == "completed" and json.loads(run["results_json"])["steps_completed"] == 6
  tr.close()


def test_hybrid_routing_model_uses_same_index_proxy():
  from nmoe_b200.parallel.hybrid import Hop, route, simulate_dispatch
  assert route(3, 3, 8) == [Hop(3, 3, "local")]
  assert route(1, 6, 8) == [Hop(1, 6, "peer")]
  assert route(1, 14, 8) == [Hop(1, 9, "net"), Hop(9, 14, "peer")]       # node 1's GPU with local index 1 forwards
  assert route(6, 14, 8) == [Hop(6, 14, "net")]                          # the proxy is the owner itself
  eid = [[0, 5, 9, 15], [3, 3, 12, 8], [1, 14, 7, 2], [6, 10, 11, 13]]   # 4 ranks, 2 per node, 16 experts (4 per rank)
  inbox, carried = simulate_dispatch(eid, 16, 4, 2)
  assert sum(len(v) for v in inbox.values()) == 16
  assert [t[2] for t in inbox[0]] == sorted(t[2] for t in inbox[0]) and all(e // 4 == 0 for _, _, e in inbox[0])
  assert carried["net"] == sum(1 for r in range(4) for e in eid[r] if (e // 4) // 2 != r // 2)


def test_loader_batches_do_not_alias_staging_buffers():
  """Batches of consecutive steps must stay distinct objects with their own contents even though the loader
  stages them through a small ring of reused host buffers."""
  from nmoe_b200.data.loader import SyntheticLoader
  ld = SyntheticLoader(vocab_size=1000, eos_token_id=999, batch_per_rank=2, seq_len=16, rank=0, seed=3, device="cpu")
  kept = [ld.next()[0].clone() for _ in range(7)]
  ld2 = SyntheticLoader(vocab_size=1000, eos_token_id=999, batch_per_rank=2, seq_len=16, rank=0, seed=3, device="cpu")
  held = [ld2.next()[0] for _ in range(7)]      # no clone: must still hold each step's own tokens afterwards
  for a, b in zip(kept, held):
    assert torch.equal(a, b)
  assert len({h.data_ptr() for h in held}) == 7


@pytest.mark.gpu
def test_loader_async_copies_see_their_own_step():
  """Several steps without any host synchronisation: every device batch equals the host sequence of its step."""
  from nmoe_b200.data.loader import SyntheticLoader
  dev = torch.device("cuda", 0)
  ld = SyntheticLoader(vocab_size=50000, eos_token_id=49999, batch_per_rank=8, seq_len=4096, rank=0, seed=5, device=dev)
  ref = SyntheticLoader(vocab_size=50000, eos_token_id=49999, batch_per_rank=8, seq_len=4096, rank=0, seed=5, device="cpu")
  big = torch.empty(1 << 28, dtype=torch.uint8, device=dev)
  got = []
  for _ in range(8):
    big.zero_(); big.add_(1)            # keep the stream busy so the copies queue up behind device work
    got.append(ld.next()[0])
  torch.cuda.synchronize()
  for g in got:
    assert torch.equal(g.cpu(), ref.next()[0])


def test_latched_kernel_status_blocks_the_checkpoint(tmp_path):
  """A status record left by a kernel (a wait that ran out, dropped rows) must stop the checkpoint before any file
  of the step exists; the record is cleared by the raise, so the next attempt goes through."""
  from nmoe_b200.checkpoint import Checkpointer, iteration_dir, read_tracker, save_checkpoint
  from nmoe_b200.data.loader import build_loader
  from nmoe_b200.ops import _lib as L
  from nmoe_b200.ops import tc_gemm
  from nmoe_b200.train import Trainer
  cfg = _tiny_cfg(tmp_path)
  dev = torch.device("cpu")
  tr = Trainer(cfg, device=dev)
  loader, plan = build_loader(cfg, 0, 1, print_fn=lambda *a: None)
  ck = Checkpointer(cfg.checkpoint_dir, async_io=False)
  tc_gemm._STATUS[dev] = torch.tensor([2, 420, 1, 7], dtype=torch.int32)
  try:
    with pytest.raises(L.NativeLibraryError, match="code=2 where=420"):
      save_checkpoint(ck, 3, tr, loader, plan, cfg, 0, C.fingerprint(cfg), print_fn=lambda *a: None, force=True)
    assert not iteration_dir(cfg.checkpoint_dir, 3).exists() and read_tracker(cfg.checkpoint_dir) == -1
    assert save_checkpoint(ck, 3, tr, loader, plan, cfg, 0, C.fingerprint(cfg), print_fn=lambda *a: None, force=True)
    assert read_tracker(cfg.checkpoint_dir) == 3
  finally:
    tc_gemm._STATUS.pop(dev, None)
    ck.close()


def test_status_watch_reports_one_step_late_without_blocking():
  from nmoe_b200.ops import _lib as L
  from nmoe_b200.ops import tc_gemm
  dev = torch.device("cpu")
  tc_gemm._STATUS[dev] = torch.zeros(4, dtype=torch.int32)
  try:
    w = tc_gemm.StatusWatch(dev, depth=2)
    for _ in range(5):
      w.poll(); w.enqueue()
    tc_gemm._STATUS[dev][:] = torch.tensor([1, 500, 3, 9], dtype=torch.int32)
    w.poll(); w.enqueue()                       # the failing step's record is only copied here ...
    with pytest.raises(L.NativeLibraryError, match="where=500"):
      w.poll()                                  # ... and seen at the next step
    assert int(tc_gemm._STATUS[dev][0]) == 0
  finally:
    tc_gemm._STATUS.pop(dev, None)


def test_nvshmem_transport_library_builds_and_exports_its_entry_points():
  """Where an NVSHMEM installation exists, the inter-node transport compiles (relocatable device code, device link
  against libnvshmem_device.a) and exports the dispatch / wait / return entry points next to the bootstrap ones."""
  import ctypes
  from nmoe_b200 import _build
  if _build.nvshmem_home() is None:
    pytest.skip("no NVSHMEM installation on this machine")
  lib = _build.build_hybrid()
  assert lib is not None and lib.exists()
  h = ctypes.CDLL(str(lib))
  for name in ("nmoe_hybrid_available", "nmoe_hybrid_uid_bytes", "nmoe_hybrid_get_uid", "nmoe_hybrid_init",
               "nmoe_hybrid_alloc", "nmoe_hybrid_free", "nmoe_hybrid_dispatch", "nmoe_hybrid_wait",
               "nmoe_hybrid_return", "nmoe_hybrid_quiet", "nmoe_hybrid_barrier", "nmoe_hybrid_finalize"):
    assert hasattr(h, name), name
  assert h.nmoe_hybrid_available() == 1 and h.nmoe_hybrid_uid_bytes() >= 64
  # before initialisation every call that needs the runtime refuses instead of touching it
  assert h.nmoe_hybrid_quiet(None) == -1 and h.nmoe_hybrid_alloc(ctypes.c_size_t(16), None) == -1


def test_zero2_buckets_walk_parameters_backwards_and_pin_the_checkpoint_layout():
  import torch
  from nmoe_b200.config import Config
  from nmoe_b200.parallel.zero2 import Zero2, bucketize
  ps = [torch.nn.Parameter(torch.zeros(n)) for n in (10, 20, 30, 40, 5)]
  b = bucketize([{"name": "dense_decay", "params": ps, "lr": 1.0, "weight_decay": 0.0}], 45)
  assert [[p.numel() for p in g["params"]] for g in b] == [[5, 40], [30, 20], [10]]
  assert all(g["name"] == "dense_decay" for g in b)
  assert bucketize([{"name": "x", "params": ps}], 0)[0]["params"] is ps
  # on CPU overlap is refused (no streams), the layout is recorded, and a foreign layout is rejected on load
  cfg = Config(dim=8, n_layers=1, n_heads=1)
  cfg.zero2_overlap = True
  z = Zero2([{"name": "dense_decay", "params": ps, "lr": 1e-2, "weight_decay": 0.0}], cfg)
  assert not z.overlap and len(z.groups) == 1
  sd = z.state_dict()
  assert sd["zero2_layout"]["bucket_elems"] == 0
  z.load_state_dict(sd)
  sd["zero2_layout"] = {"bucket_elems": 123, "totals": [1]}
  import pytest
  with pytest.raises(ValueError, match="layout"):
    z.load_state_dict(sd)


def test_checkpoint_write_timing_interval_hint_and_run_info(tmp_path, monkeypatch):
  from nmoe_b200.checkpoint import Checkpointer, read_latest_run_info
  from nmoe_b200.train import train
  ck = Checkpointer(str(tmp_path / "plain"), async_io=False)
  assert ck.recommend_interval(400.0) == 1                       # nothing timed yet
  ck.submit(tmp_path / "plain" / "iter_0000001" / "dp_rank_000.pt", {"step": 1, "w": torch.zeros(4)}, 1, 1)
  assert ck.last_write_ms > 0 and ck.last_stage_ms >= 0
  ck.last_write_ms = 9000.0                                      # a 9 s save against 400 ms steps
  assert ck.recommend_interval(400.0) == 30 and ck.recommend_interval(400.0, safety=1.0) == 23
  assert ck.recommend_interval(0.0) == 1
  ck.close()
  assert read_latest_run_info(tmp_path / "none") is None
  monkeypatch.setenv("NMOE_RUN", "info")
  cfg = _tiny_cfg(tmp_path / "r")
  train(cfg)
  info = read_latest_run_info(cfg.checkpoint_dir)
  assert info["step"] == 6 and info["tokens"] == 6 * cfg.batch_size * cfg.seq_len and info["E"] == cfg.n_routed_experts


def test_dispatch_counters_follow_the_polled_row_counts(capsys):
  """``Rdep.comm_counters`` reports what ``_poll_seen`` has learnt from pinned memory; no device is involved."""
  import collections
  from nmoe_b200.parallel.rdep import Rdep
  r = Rdep.__new__(Rdep)
  r.rank, r.capacity, r._rows_hwm, r._rows_grain = 0, 8192, 4096, 4096
  r.rows_overflows = r.rows_last = r.rows_dropped = 0
  r._seen = torch.tensor([20, -1, 40], dtype=torch.int32)            # tiles of 128 rows; -1 = that kernel has not run yet
  r._seen_pending = collections.deque([(0, 32), (2, 32), (1, 32)])
  r._poll_seen()
  c = r.comm_counters()
  assert c["M_recv"] == 5120 and c["dropped_rows"] == 1024 and c["overflow_calls"] == 1 and c["capacity_utilization"] == 0.625
  assert c["row_bound"] == 8192 and list(r._seen_pending) == [(1, 32)]
  assert "1024 rows of that call were not computed" in capsys.readouterr().err


def test_param_summary_counts_experts_of_all_ranks(tmp_path):
  from nmoe_b200.metrics import param_counts, param_summary
  from nmoe_b200.train import Trainer
  cfg = _tiny_cfg(tmp_path)
  m = Trainer(cfg).model
  n = sum(p.numel() for p in m.parameters())
  experts = sum(p.numel() for p in m.param_sets()[0])
  total, active = param_counts(m, cfg, 1)
  assert total == n and active == n - experts + experts * cfg.n_activated_experts // cfg.n_routed_experts
  assert param_counts(m, cfg, 4)[0] == n + 3 * experts
  assert param_summary(m, cfg).startswith("(0.00B params")


def test_step_profiler_writes_trace_and_operator_table(tmp_path, monkeypatch):
  """profiling_enabled: the configured steps are recorded with the module scopes switched on only meanwhile."""
  from nmoe_b200.train import train
  from nmoe_b200.utils import profiling as P
  monkeypatch.setenv("NMOE_RUN", "prof")
  cfg = _tiny_cfg(tmp_path, steps=7, checkpoint_every=100, profiling_enabled=True, profiling_steps=2, profiling_skip=1,
                  profiling_output_dir=str(tmp_path / "profiles"))
  assert not P.scopes_enabled() and P.scope("x") is P.scope("y")           # off: one shared do-nothing context
  train(cfg)
  assert not P.scopes_enabled()
  d = tmp_path / "profiles" / "prof"
  trace = json.loads((d / "trace_rank0.json").read_text())
  names = {e.get("name") for e in trace["traceEvents"]}
  assert {"embed", "block_00/attn_global", "block_00/mlp", "block_01/moe", "lm_head_loss", "backward", "optimizer"} <= names
  assert sum(1 for e in trace["traceEvents"] if e.get("name") == "lm_head_loss" and e.get("ph") == "X") == 2      # two active steps
  assert "Self CPU" in (d / "ops_rank0.txt").read_text()
  # a run that ends inside the profile still leaves its files; a disabled profiler does nothing
  pr = P.StepProfiler(True, tmp_path / "cut", steps=5, skip=0, print_fn=lambda *_: None)
  for _ in range(3):
    with P.scope("work"):
      torch.ones(4).sum()
    pr.step()
  pr.close()
  assert pr.done and (tmp_path / "cut" / "trace_rank0.json").exists() and not P.scopes_enabled()
  off = P.StepProfiler(False, tmp_path / "off")
  off.step(); off.close()
  assert off.done and not (tmp_path / "off").exists()


def test_reference_module_paths_are_aliases_that_cannot_shadow_another_install():
  """`python -m nmoe.train / nmoe.data.cli / nmoe.eval.*` resolve to this package; the alias tree has no __init__.py
  anywhere, so a regular `nmoe` package found later on sys.path (the reference, when it is installed) still wins."""
  import importlib
  import subprocess
  import sys
  from pathlib import Path
  root = Path(__file__).resolve().parent.parent
  assert not list((root / "nmoe").rglob("__init__.py"))
  import nmoe_b200.data.cli, nmoe_b200.eval.runner, nmoe_b200.train
  sys.path.insert(0, str(root))
  try:
    assert importlib.import_module("nmoe.train").main is nmoe_b200.train.main
    assert importlib.import_module("nmoe.data.cli").main is nmoe_b200.data.cli.main
    assert importlib.import_module("nmoe.eval.runner").main is nmoe_b200.eval.runner.main
    assert importlib.import_module("nmoe.eval.choices").run_eval is importlib.import_module("nmoe_b200.eval.choices").run_eval
  finally:
    sys.path.remove(str(root))
  out = subprocess.run([sys.executable, "-m", "nmoe.data.cli", "info", "--help"], cwd=root, capture_output=True, text=True)
  assert out.returncode == 0 and "usage" in out.stdout


def test_sigusr1_stops_at_a_checkpoint_and_the_restart_finishes_the_same_run(tmp_path, monkeypatch):
  """A stop request between steps: checkpoint of that step, run recorded as killed; the restarted job resumes from it
  and ends with the loss of a run that was never interrupted."""
  import os
  import signal
  import nmoe_b200.train as T
  from nmoe_b200.checkpoint import read_tracker
  from nmoe_b200.experiments import ExperimentTracker
  monkeypatch.setenv("NMOE_RUN", "whole")
  whole = T.train(_tiny_cfg(tmp_path / "a", checkpoint_every=100))
  import nmoe_b200.metrics as M
  real_log = M.log_training_step
  def log_and_signal(metrics, s, *a, **kw):
    if s == 3:
      os.kill(os.getpid(), signal.SIGUSR1)
    return real_log(metrics, s, *a, **kw)
  monkeypatch.setattr(M, "log_training_step", log_and_signal)
  monkeypatch.setenv("NMOE_RUN", "cut")
  before = signal.getsignal(signal.SIGUSR1)
  cfg = _tiny_cfg(tmp_path / "b", checkpoint_every=100)
  part = T.train(cfg)
  assert part["steps_completed"] == 3 and read_tracker(cfg.checkpoint_dir) == 3
  assert signal.getsignal(signal.SIGUSR1) == before                       # handlers are put back
  tr = ExperimentTracker(cfg)
  assert tr.get_run("cut").status == "killed" and json.loads(tr.get_run("cut").results_json)["steps_completed"] == 3
  tr.close()
  monkeypatch.setattr(M, "log_training_step", real_log)
  rest = T.train(_tiny_cfg(tmp_path / "b", checkpoint_every=100))
  assert rest["steps_completed"] == 6 and rest["final_loss"] == whole["final_loss"] and rest["tokens_seen"] == whole["tokens_seen"]
  tr = ExperimentTracker(cfg)
  assert tr.get_run("cut").status == "completed"
  tr.close()


def test_stop_request_agreement_logic_single_rank():
  from nmoe_b200.utils.stop import StopRequest
  s = StopRequest(1, install=False)
  assert not s.should_stop(1) and not s.should_stop(2)
  s.request("operator")
  assert s.should_stop(3) and s.stop_at == 3 and s.reason == "operator" and s.should_stop(4)


def test_every_shipped_config_loads_with_its_loader():
  import glob
  from pathlib import Path
  from nmoe_b200.config import from_toml, load_toml
  from nmoe_b200.data.flow import load_spec
  from nmoe_b200.data.mixture import resolve_plan
  from nmoe_b200.data.registry import Registry
  models = [f for f in sorted(glob.glob("configs/*.toml")) if not f.endswith(("flow_profiles.toml", "tasks.toml"))]
  assert len(models) >= 6
  for f in models:
    cfg = from_toml(f, [], env={})
    cfg.validate(1)
    if cfg.batch_size % 8 == 0:
      cfg.validate(8)
  for f in glob.glob("configs/**/*.toml", recursive=True):
    load_toml(f)
  flows = load_toml("configs/flow_profiles.toml")
  for name, prof in flows["profiles"].items():
    plan = resolve_plan(mixture_toml=Path(prof["mixture"]), flow_profiles_toml=Path("configs/flow_profiles.toml"),
                        flow_section=f"flow.{prof['flow']}", seq_len=4096, active_params_b=3.0)
    assert plan.stages and plan.stages[0].sources, name
  for f in glob.glob("configs/dataflow/*.toml"):
    assert load_spec(Path(f), env={}).prep["output_dir"]
  assert Registry.load("configs/tasks.toml").tasks


def test_second_stop_signal_is_not_intercepted():
  """The first SIGUSR1 asks for a checkpointed stop; the second gets the disposition the process had before."""
  import os
  import signal
  from nmoe_b200.utils.stop import StopRequest
  hits = []
  before = signal.signal(signal.SIGUSR1, lambda s, f: hits.append(s))
  try:
    st = StopRequest(1, signals=(signal.SIGUSR1,))
    os.kill(os.getpid(), signal.SIGUSR1)
    assert st.requested and st.reason == "SIGUSR1" and hits == []
    os.kill(os.getpid(), signal.SIGUSR1)
    assert hits == [signal.SIGUSR1]                         # went to the handler that was there before
    os.kill(os.getpid(), signal.SIGUSR1)
    assert len(hits) == 2 and st.should_stop(1)
  finally:
    signal.signal(signal.SIGUSR1, before)


def test_train_entry_point_overrides_and_errors(tmp_path, monkeypatch, capsys):
  """`python -m nmoe_b200.train cfg.toml --key=value`: precedence TOML < NMOE_* < flags, unknown keys refused, a failed
  run recorded as failed."""
  import nmoe_b200.train as T
  from nmoe_b200.experiments import ExperimentTracker
  cfg = _tiny_cfg(tmp_path)
  toml = tmp_path / "c.toml"
  import dataclasses
  keep = {k: v for k, v in dataclasses.asdict(cfg).items() if not k.startswith("_") and v is not None and not isinstance(v, dict)}
  toml.write_text("".join(f"{k} = {json.dumps(v)}\n" for k, v in keep.items()))
  monkeypatch.setenv("NMOE_RUN", "cli")
  monkeypatch.setenv("NMOE_STEPS", "5")                       # environment beats the file ...
  T.main([str(toml), "--steps=2", "--log_every", "1"])         # ... and the flag beats the environment
  out = capsys.readouterr().out
  assert "step      2" in out and "step      3" not in out and "Training complete" in out
  with pytest.raises(TypeError):
    T.main([str(toml), "--no_such_key=1"])
  with pytest.raises(SystemExit):
    T.main([])
  # a run that dies is recorded as failed, and the error reaches the caller
  monkeypatch.setenv("NMOE_RUN", "dies")
  import nmoe_b200.metrics as M
  def boom(*a, **k):
    raise RuntimeError("injected")
  monkeypatch.setattr(M, "log_training_step", boom)
  with pytest.raises(RuntimeError, match="injected"):
    T.main([str(toml), "--steps=2", "--resume=false", f"--checkpoint_dir={tmp_path / 'ck2'}"])
  tr = ExperimentTracker(cfg)
  assert tr.get_run("dies").status == "failed" and tr.get_run("cli").status == "completed"
  tr.close()
