"""End-to-end training on one GPU through the public loop (`train(cfg)`): the loss of a small Moonlight-shaped model
(MLA attention, routed + shared experts, fp8 expert GEMMs) must fall over a few dozen steps at a real learning rate,
and the per-module / collective timers must land in the metrics store."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _cfg(tmp_path, **kw):
  from nmoe_b200.config import Config
  base = dict(vocab_size=2048, eos_token_id=2047, dim=512, n_layers=2, n_heads=4, inter_dim=1024, moe_inter_dim=256,
              n_routed_experts=8, n_activated_experts=2, n_shared_experts=2, n_dense_layers=1, q_lora_rank=256,
              kv_lora_rank=128, qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128, route_scale=2.446,
              batch_size=4, seq_len=256, max_position_embeddings=512, warmup_steps=5, steps=30, log_every=5,
              lr_dense=2e-3, lr_router=2e-3, lr_expert=2e-3, checkpoint_every=1000, resume=False, data_path="synthetic",
              checkpoint_dir=str(tmp_path / "ckpt"), metrics_dir=str(tmp_path / "metrics"),
              experiments_db=str(tmp_path / "exp.db"))
  base.update(kw)
  return Config(**base)


@pytest.mark.parametrize("dtype", ["bf16", "fp8"])
def test_loss_falls_on_a_moonlight_shaped_model(tmp_path, monkeypatch, dtype):
  from nmoe_b200.metrics import MetricsWriter
  from nmoe_b200.ops import tc_gemm as G
  from nmoe_b200.train import train
  monkeypatch.setenv("NMOE_RUN", f"gpu_{dtype}")
  cfg = _cfg(tmp_path, dtype=dtype)

  # a fixed, learnable stream: the same 4 sequences every step (the synthetic loader draws new noise per step)
  import nmoe_b200.data.loader as LD

  class Repeat(LD.SyntheticLoader):
    def next_host(self):
      self.step = 0
      return super().next_host()
  monkeypatch.setattr(LD, "SyntheticLoader", Repeat)

  res = train(cfg)
  G.check_status()
  w = MetricsWriter(f"gpu_{dtype}", cfg.metrics_dir, 0)
  loss = [v for _, v in w.query("train/loss")]
  assert len(loss) >= 5 and all(math.isfinite(v) for v in loss)
  assert loss[0] > 7.0                       # ~ ln(vocab) at the start
  assert loss[-1] < loss[0] - 1.0, loss      # memorising four sequences: a right backward brings it down fast
  assert res["steps_completed"] == 30
  tags = {t for (t,) in w.db.execute("select distinct tag from metrics").fetchall()} if hasattr(w, "db") else set()
  if tags:
    assert any("attn_fwd" in t for t in tags) and any("moe_bwd" in t for t in tags), sorted(tags)[:40]
  w.close()


def test_dense_updates_issued_from_backward_hooks_match_the_step_after_backward(tmp_path):
  """ZeRO-2 overlap on one GPU: the dense parameters are cut into buckets and every bucket's AdamW is queued on a side
  stream as soon as backward has written its last gradient.  (a) With exactly reproducible gradients (loss = sum p*c)
  the parameters equal, bit for bit, those of the same buckets stepped after backward.  (b) A whole model trains to
  the same loss curve either way (its own reductions are not bitwise repeatable, so the curve is compared)."""
  from nmoe_b200.config import Config
  from nmoe_b200.ops import tc_gemm as G
  from nmoe_b200.parallel.zero2 import Zero2
  from nmoe_b200.train import Trainer
  dev = torch.device("cuda")
  cfg0 = Config(dim=8, n_layers=1, n_heads=1)
  cfg0.zero2_overlap, cfg0.zero2_bucket_mb = True, 0.05
  res = {}
  for from_hooks in (False, True):
    g = torch.Generator().manual_seed(3)
    params = [torch.nn.Parameter(torch.randn(n, generator=g).bfloat16().to(dev)) for n in (1000, 40960, 77, 130000, 512, 30000)]
    z = Zero2([{"name": "dense_decay", "params": params[:4], "lr": 1e-2, "weight_decay": 0.1},
               {"name": "router", "params": params[4:], "lr": 5e-3, "weight_decay": 0.0}], cfg0)
    assert z.impl == "single" and z.overlap and len(z.groups) >= 4
    for step in range(3):
      z.zero_grad()
      if not from_hooks:
        z._armed = False
      gg = torch.Generator().manual_seed(100 + step)
      loss = sum((p * (torch.randn(p.numel(), generator=gg) * 0.1).bfloat16().to(dev).view_as(p)).sum() for p in params)
      loss.backward()
      assert all(g_.launched for g_ in z.groups) == from_hooks
      z.step()
    torch.cuda.synchronize()
    res[from_hooks] = torch.cat([p.detach().float().cpu().view(-1) for p in params])
  assert torch.equal(res[False], res[True])

  losses = []
  for overlap in (False, True):
    cfg = _cfg(tmp_path, dtype="bf16", zero2_overlap=overlap, zero2_bucket_mb=1)
    torch.manual_seed(5)
    tr = Trainer(cfg, rank=0, world=1, device=dev, fuse_expert_opt=False)
    assert tr.opt.dense.overlap == overlap and (len(tr.opt.dense.groups) > 3) == overlap
    g = torch.Generator().manual_seed(9)
    tok = torch.randint(0, 2000, (4, 257), generator=g)
    x, y = tok[:, :-1].contiguous().to(dev), tok[:, 1:].contiguous().to(dev)
    losses.append([float(tr.step(x, y).item()) for _ in range(6)])
    torch.cuda.synchronize()
    G.check_status()
  for a, b in zip(*losses):
    assert abs(a - b) <= 2e-3 * abs(a), losses
  assert losses[1][-1] < losses[1][0] - 0.3, losses


def test_expert_updates_on_a_side_stream_train_like_updates_on_the_compute_stream(tmp_path, monkeypatch):
  """The in-backward expert AdamW runs on its own stream so that it overlaps the backward GEMMs of the layers below;
  ordering is by events only.  Same loss curve as with everything on one stream (a raced update would not give it),
  and the side stream is joined before the step returns."""
  from nmoe_b200.ops import tc_gemm as G
  from nmoe_b200.train import Trainer
  dev = torch.device("cuda")
  curves = []
  for side in ("0", "1"):
    monkeypatch.setenv("NMOE_EXPERT_OPT_SIDE_STREAM", side)
    cfg = _cfg(tmp_path, dtype="fp8", n_layers=3)
    torch.manual_seed(5)
    tr = Trainer(cfg, rank=0, world=1, device=dev)
    assert (tr.opt.expert.side is not None) == (side == "1")
    g = torch.Generator().manual_seed(9)
    tok = torch.randint(0, 2000, (4, 257), generator=g)
    x, y = tok[:, :-1].contiguous().to(dev), tok[:, 1:].contiguous().to(dev)
    ls = []
    for _ in range(10):
      ls.append(float(tr.step(x, y).item()))
    torch.cuda.synchronize()
    G.check_status()
    curves.append(ls)
  for a, b in zip(*curves):
    assert abs(a - b) <= 5e-3 * abs(a), curves
  assert curves[1][-1] < curves[1][0] - 0.5, curves
