"""Toy MoE transformer in fp32 on CPU (the numerical oracle configuration): one
forward/backward/AdamW step, checked against independent eager statements of the math."""
import math

import torch
import torch.nn.functional as F

from nmoe_b200.config import Config
from nmoe_b200.train import Trainer


def toy_cfg(**kw):
  base = dict(vocab_size=1024, eos_token_id=1023, dim=256, n_layers=4, n_heads=4, inter_dim=1024, moe_inter_dim=128,
              n_routed_experts=8, n_activated_experts=2, n_shared_experts=1, n_dense_layers=1, q_lora_rank=96,
              kv_lora_rank=64, qk_nope_head_dim=32, qk_rope_head_dim=16, v_head_dim=32, batch_size=2, seq_len=128,
              max_position_embeddings=256, warmup_steps=1, lr_dense=3e-3, lr_expert=3e-3, lr_router=3e-3,
              activation_checkpoint="none")
  base.update(kw)
  return Config(**base)


def test_one_step_and_loss_decreases():
  torch.manual_seed(0)
  cfg = toy_cfg()
  tr = Trainer(cfg)
  tok = torch.randint(0, cfg.vocab_size - 1, (2, 129))
  x, y = tok[:, :-1], tok[:, 1:]
  l0 = tr.step(x, y).item()
  assert math.isfinite(l0) and abs(l0 - math.log(cfg.vocab_size)) < 1.5
  for _ in range(5):
    l = tr.step(x, y).item()
  assert l < l0 - 0.05, (l0, l)


def test_moe_layer_matches_per_token_loop():
  torch.manual_seed(1)
  cfg = toy_cfg()
  tr = Trainer(cfg)
  moe = tr.model.blocks[1].ffn
  X = torch.randn(16, cfg.dim) * 0.5
  out = moe(X)
  # independent statement: per token, per selected expert
  logits = X @ moe.router.gate.t() * cfg.route_scale
  s = torch.sigmoid(logits)
  idx = torch.topk(s + moe.router.bias, cfg.n_activated_experts, dim=-1).indices
  ref = torch.zeros_like(X)
  for t in range(X.size(0)):
    w = s[t, idx[t]]
    w = w / w.sum()
    for k, e in enumerate(idx[t].tolist()):
      h = X[t] @ moe.W13[e].t()
      a = F.silu(h[0::2]) * h[1::2]
      ref[t] += w[k] * (a @ moe.W2[e].t())
    hs = X[t] @ moe.shared.w13.t()
    ref[t] += (F.silu(hs[0::2]) * hs[1::2]) @ moe.shared.w2.t()
  assert torch.allclose(out, ref, atol=1e-5, rtol=1e-4)


def test_mla_matches_eager_reference_math():
  """Same composition as nmoe/attention/mla.py:178-197 written with plain tensor ops."""
  torch.manual_seed(2)
  cfg = toy_cfg()
  tr = Trainer(cfg)
  m = tr.model.blocks[0].attn
  x = torch.randn(2, 20, cfg.dim)
  cos, sin = tr.model.rope.cos[:20], tr.model.rope.sin[:20]
  out = m(x, cos, sin)

  def rms(v, w):
    return v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + cfg.rms_norm_eps) * w

  def rot(v):
    c, s_ = cos.unsqueeze(-2), sin.unsqueeze(-2)
    h = v.size(-1) // 2
    return torch.cat((v[..., :h] * c - v[..., h:] * s_, v[..., h:] * c + v[..., :h] * s_), -1)

  B, S, H = 2, 20, cfg.n_heads
  q = (rms(x @ m.wq_a.t(), m.q_norm.weight) @ m.wq_b.t()).view(B, S, H, -1)
  qn, qp = q[..., :32], rot(q[..., 32:])
  kva = x @ m.wkv_a.t()
  kp = rot(kva[..., 64:].unsqueeze(2))
  kv = (rms(kva[..., :64], m.kv_norm.weight) @ m.wkv_b.t()).view(B, S, H, 64)
  kn, v = kv[..., :32], kv[..., 32:]
  qq = torch.cat((qn, qp), -1)
  kk = torch.cat((kn, kp.expand(B, S, H, 16)), -1)
  sc = torch.einsum("bihd,bjhd->bhij", qq, kk) * (48 ** -0.5)
  sc = sc.masked_fill(torch.triu(torch.ones(S, S, dtype=torch.bool), 1), float("-inf"))
  o = torch.einsum("bhij,bjhd->bihd", sc.softmax(-1), v).reshape(B, S, -1) @ m.wo.t()
  assert torch.allclose(out, o, atol=1e-5, rtol=1e-4)


def test_local_global_interleave_and_swa():
  cfg = toy_cfg(attn_global_every=3, attn_local_window=16, n_layers=7)
  kinds = [cfg.is_global_layer(i) for i in range(7)]
  assert kinds == [False, False, True, False, False, True, True]
  torch.manual_seed(3)
  tr = Trainer(cfg)
  names = [type(b.attn).__name__ for b in tr.model.blocks]
  assert names == ["SWA", "SWA", "MLA", "SWA", "SWA", "MLA", "MLA"]
  tok = torch.randint(0, 1000, (2, 129))
  assert math.isfinite(tr.step(tok[:, :-1], tok[:, 1:]).item())


def test_masked_loss_ignores_eos_targets():
  torch.manual_seed(4)
  cfg = toy_cfg(n_layers=2)
  tr = Trainer(cfg)
  tok = torch.randint(0, 1000, (2, 129))
  y = tok[:, 1:].clone()
  with torch.no_grad():
    base = tr.model.loss(tok[:, :-1], y)
    logits = tr.model(tok[:, :-1])
    y2 = y.clone()
    y2[:, ::2] = cfg.eos_token_id
    masked = tr.model.loss(tok[:, :-1], y2)
    per = F.cross_entropy(logits.reshape(-1, cfg.vocab_size), y.reshape(-1), reduction="none").view(2, 128)
  assert torch.allclose(base, per.mean(), atol=1e-5)
  assert torch.allclose(masked, per[:, 1::2].mean(), atol=1e-5)


def test_muon_expert_optimizer_cpu():
  from nmoe_b200.ops.muon import Muon, newton_schulz
  torch.manual_seed(6)
  w = torch.nn.Parameter(torch.randn(2, 16, 32))
  y = newton_schulz(w.detach())
  s = torch.linalg.svdvals(y)
  assert s.max() < 1.3 and s.min() > 0.5
  opt = Muon([w], lr=0.1, momentum=0.9)
  target = torch.randn(2, 16, 32)
  l0 = None
  for _ in range(20):
    loss = (w - target).pow(2).mean()
    l0 = l0 or loss.item()
    loss.backward()
    opt.step()
  assert loss.item() < l0


def test_trunc_normal_init_has_no_outliers_in_bf16():
  """Sampling happens in fp32: a bf16 weight must not pick up the +-2 outliers that the stock
  low-precision ``trunc_normal_`` produces."""
  import torch
  from nmoe_b200.models.init import trunc_normal_
  torch.manual_seed(0)
  w = torch.empty(64, 2048, dtype=torch.bfloat16)
  trunc_normal_(w, std=0.02)
  assert w.float().abs().max().item() < 0.02 * 6.5
  assert abs(w.float().std().item() - 0.02) < 1e-3
  w2 = torch.empty(4096, dtype=torch.float32)
  trunc_normal_(w2, std=1.0, a=-1.0, b=1.0)
  assert w2.abs().max().item() <= 1.0
