"""The interactive toolkit on a tiny CPU model: memory tables, phase timing, router probe, gradient report, checkpoint
inspection, quick ablation runs."""
import math

import torch

from nmoe_b200 import lab


def test_param_tables_match_the_model_and_the_analytic_count():
  t = lab.tiny_trainer()
  rows = lab.param_memory(t.model)
  total = rows[-1]
  n = sum(p.numel() for p in t.model.parameters())
  assert total["group"] == "total" and abs(total["params_m"] * 1e6 - n) < 1 and total["tensors"] == len(list(t.model.parameters()))
  by = {r["group"]: r for r in rows}
  assert {"routed experts", "attention", "embeddings", "norms", "router", "shared experts"} <= set(by)
  experts = sum(p.numel() for name, p in t.model.named_parameters() if name.endswith((".W13", ".W2")))
  assert abs(by["routed experts"]["params_m"] * 1e6 - experts) < 1
  counted = lab.count_params(t.cfg)
  assert counted["expert"] == experts and counted["dense"] == n - experts
  est1, est8 = lab.training_state_estimate(t.cfg, 1), lab.training_state_estimate(t.cfg, 8)
  assert est8["expert_weights_gib"] * 8 == est1["expert_weights_gib"] and est8["dense_weights_gib"] == est1["dense_weights_gib"]
  assert est8["total_gib"] < est1["total_gib"]
  text = lab.show(rows, print_fn=lambda *_: None)
  assert text.splitlines()[0].split() == ["group", "tensors", "params_m", "mib"] and "routed experts" in text
  assert set(lab.mem_stats()) == {"allocated_gib", "reserved_gib", "peak_gib", "free_gib", "total_gib"}


def test_time_step_router_probe_and_gradient_report():
  t = lab.tiny_trainer(n_layers=3)
  tm = lab.time_step(t, warmup=1, iters=2)
  assert all(tm[k] > 0 for k in ("forward_ms", "backward_ms", "optimizer_ms")) and tm["tokens_per_s"] > 0
  assert abs(tm["total_ms"] - tm["forward_ms"] - tm["backward_ms"] - tm["optimizer_ms"]) < 1e-9
  with lab.RouterProbe(t.model) as probe:
    losses = lab.run_steps(t, 4)
  assert len(probe.history) == 4 and losses[-1] < losses[0]
  lab.run_steps(t, 1)
  assert len(probe.history) == 4                          # the hook is gone after the block
  tot = probe.total()
  picks = t.cfg.batch_size * t.cfg.seq_len * t.cfg.n_activated_experts
  assert tot.shape == (2, t.cfg.n_routed_experts) and torch.all(tot.sum(-1) == 4 * picks)
  rows = probe.table()
  assert [r["moe_layer"] for r in rows] == [0, 1]
  for r in rows:
    assert 0 <= r["cv"] and r["experts_active"] + r["dead"] == t.cfg.n_routed_experts and r["hottest_share"] >= r["ideal_share"]
  assert len(probe.drift()) == 3 and all(0 <= d <= 1 for d in probe.drift())

  loss = lab.backward_only(t)
  rep = lab.grad_report(t.model)
  blocks = {r["block"] for r in rep}
  assert {"blocks.00.attn", "blocks.01.ffn", "embedding", "lm_head"} <= blocks and math.isfinite(loss)
  assert all(r["non_finite"] == 0 and r["no_grad"] == 0 and r["grad_norm"] > 0 for r in rep)
  # a poisoned gradient is counted
  t.model.lm_head.grad[0, 0] = float("nan")
  assert {r["block"]: r["non_finite"] for r in lab.grad_report(t.model)}["lm_head"] == 1


def test_checkpoint_listing_and_peek(tmp_path, monkeypatch):
  from nmoe_b200.config import Config
  from nmoe_b200.train import train
  monkeypatch.setenv("NMOE_RUN", "labrun")
  cfg = Config(**{**lab._TINY, "steps": 4, "log_every": 2, "checkpoint_every": 2, "checkpoint_dir": str(tmp_path / "ck"),
                  "metrics_dir": str(tmp_path / "m"), "experiments_db": str(tmp_path / "e.db")})
  train(cfg)
  rows = lab.list_checkpoints(tmp_path / "ck")
  assert [r["step"] for r in rows] == [2, 4] and all(r["finalised"] for r in rows) and [r["latest"] for r in rows] == [False, True]
  peek = lab.peek_checkpoint(tmp_path / "ck")
  assert peek["step"] == 4 and peek["manifest"]["step"] == 4 and peek["rd"]["step"] == 4
  assert any(str(v).startswith("tensor[") for v in peek["rd"]["model_dense"].values())
  assert "model_expert" in peek["dp_rank"] and peek["dense_params_m"] > 0
  assert lab.list_checkpoints(tmp_path / "nope") == []
  import pytest
  with pytest.raises(FileNotFoundError):
    lab.peek_checkpoint(tmp_path / "empty")


def test_quick_train_compares_two_settings():
  quiet = lambda *_: None
  a = lab.quick_train({"lr_dense": 3e-3, "lr_expert": 3e-3}, steps=25, print_fn=quiet)
  b = lab.quick_train({"lr_dense": 1e-6, "lr_expert": 1e-6, "decay_floor": 1e-7}, steps=25, print_fn=quiet)
  assert len(a) == 25 and a[0] == b[0]                     # same seed, same first batch, same initial weights
  rows = {r["run"]: r for r in lab.compare({"lr 3e-3": a, "lr 1e-6": b})}
  assert rows["lr 3e-3"]["drop"] > rows["lr 1e-6"]["drop"] and rows["lr 3e-3"]["drop"] > 0.05


def test_quickstart_notebook_cells_run(tmp_path, monkeypatch):
  """Every code cell of notebooks/quickstart.ipynb executes in order in one namespace."""
  import json
  from pathlib import Path
  nb = json.loads((Path(__file__).resolve().parent.parent / "notebooks" / "quickstart.ipynb").read_text())
  monkeypatch.setenv("TMPDIR", str(tmp_path))
  import tempfile
  monkeypatch.setattr(tempfile, "tempdir", str(tmp_path))
  ns = {}
  cells = [c for c in nb["cells"] if c["cell_type"] == "code"]
  assert len(cells) >= 8
  for c in cells:
    exec(compile("".join(c["source"]), "<quickstart cell>", "exec"), ns)
  assert ns["store"].runs() == ["quickstart"] and set(ns["curves"]) == {"lr 3e-3", "lr 3e-4", "top-4"}


def test_profile_steps_lists_operators_and_scopes():
  from nmoe_b200.utils import profiling as P
  t = lab.tiny_trainer()
  rows = lab.profile_steps(t, steps=2, warmup=1, top=400)
  names = {r["name"] for r in rows}
  assert {"backward", "optimizer", "lm_head_loss", "block_01/moe"} <= names and not P.scopes_enabled()
  scope = next(r for r in rows if r["name"] == "lm_head_loss")
  assert scope["calls_per_step"] == 1.0 and all(r["host_ms_per_step"] >= 0 for r in rows)
  assert rows == sorted(rows, key=lambda r: -r["host_ms_per_step"])


def test_trainer_from_a_shipped_configuration_with_overrides():
  t = lab.trainer_from("configs/toy.toml", steps=3, batch_size=2, seq_len=32)
  assert t.cfg.preset == "toy" and t.cfg.batch_size == 2 and t.cfg.seq_len == 32
  losses = lab.run_steps(t, 3)
  assert len(losses) == 3 and all(math.isfinite(x) for x in losses)
  est = lab.training_state_estimate(t.cfg)
  assert est["total_gib"] > 0 and lab.count_params(t.cfg)["dense"] + lab.count_params(t.cfg)["expert"] == sum(p.numel() for p in t.model.parameters())
