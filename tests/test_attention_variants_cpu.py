"""NSA / DSA / KDA on CPU: oracle checks of their building blocks and end-to-end training steps."""
import math

import torch

from nmoe_b200.config import Config
from nmoe_b200.models.attention import dsa, kda
from nmoe_b200.train import Trainer


def _cfg(**kw):
  base = dict(vocab_size=512, eos_token_id=511, dim=64, n_layers=2, n_heads=4, inter_dim=128, moe_inter_dim=32,
              n_routed_experts=4, n_activated_experts=2, n_shared_experts=1, n_dense_layers=1, q_lora_rank=32,
              kv_lora_rank=16, qk_nope_head_dim=8, qk_rope_head_dim=8, v_head_dim=16, batch_size=2, seq_len=128,
              max_position_embeddings=256, warmup_steps=1, lr_dense=3e-3, lr_expert=3e-3, lr_router=3e-3,
              activation_checkpoint="none")
  base.update(kw)
  return Config(**base)


def test_kda_chunked_matches_recurrence():
  torch.manual_seed(0)
  B, T, H, Dk, Dv = 2, 150, 2, 16, 8
  q, k = torch.randn(B, T, H, Dk), torch.randn(B, T, H, Dk)
  v = torch.randn(B, T, H, Dv)
  g = torch.nn.functional.logsigmoid(torch.randn(B, T, H, Dk) + 2)
  beta = torch.sigmoid(torch.randn(B, T, H))
  ref = kda.kda_recurrent(q, k, v, g, beta)
  for chunk in (16, 64):
    out = kda.kda_chunked(q, k, v, g, beta, chunk=chunk)
    assert torch.allclose(out, ref, atol=2e-4, rtol=1e-3), (out - ref).abs().max()


def test_lightning_indexer_causal_topk():
  torch.manual_seed(1)
  q, k, w = torch.randn(1, 20, 3, 8), torch.randn(1, 20, 8), torch.randn(1, 20, 3)
  vals, idx = dsa.lightning_indexer(q, k, w, 5)
  s = (w.unsqueeze(-1) * torch.relu(torch.einsum("bmhd,bnd->bmhn", q, k))).sum(2)
  for t in range(20):
    allowed = s[0, t, :t + 1]
    kk = min(5, t + 1)
    assert set(idx[0, t, :kk].tolist()) == set(allowed.topk(kk).indices.tolist())
    assert (idx[0, t, :kk] <= t).all()


def test_dsa_full_topk_equals_mla_and_alignment_loss():
  torch.manual_seed(2)
  cfg = _cfg(attn="dsa", attn_dsa={"top_k": 4096, "n_idx_heads": 2, "idx_dim": 8})
  tr = Trainer(cfg)
  blk = tr.model.blocks[0].attn
  x = torch.randn(2, 32, cfg.dim)
  cos, sin = tr.model.rope.cos[:32], tr.model.rope.sin[:32]
  from nmoe_b200.models.attention.mla import MLA
  y = blk(x, cos, sin)
  y_mla = MLA.forward(blk, x, cos, sin)
  assert torch.allclose(y, y_mla, atol=1e-5)
  assert math.isfinite(blk.indexer_alignment_loss().item())
  blk.training_mode = "dense_warmup"
  assert torch.allclose(blk(x, cos, sin), y_mla, atol=1e-5)
  l = blk.indexer_alignment_loss()
  l.backward()
  assert blk.wq_idx.grad is not None and math.isfinite(l.item())


def test_nsa_blocks_and_training_step():
  torch.manual_seed(3)
  cfg = _cfg(attn="nsa", attn_global_every=2, attn_local="nsa", attn_local_window=32,
             attn_nsa={"cmp_len": 8, "cmp_stride": 4, "slc_block": 16, "topk_blocks": 4, "kv_heads": 2})
  tr = Trainer(cfg)
  nsa = tr.model.blocks[0].attn
  assert nsa.window == 32
  T = 128
  sc = torch.rand(1, T, 2, T // 16)
  blocks = nsa.select_blocks(sc, T)
  t = 100
  assert blocks[0, t, 0, 0] == 0 and set(blocks[0, t, 0, 1:3].tolist()) == {4, 5} and (blocks[0, t] < 7).all()
  xk = torch.randn(1, 30, 2, 16)
  assert nsa.compress(xk).shape == (1, (30 - 8) // 4 + 1, 2, 16)
  tok = torch.randint(0, 500, (2, 129))
  l0 = tr.step(tok[:, :-1], tok[:, 1:]).item()
  for _ in range(4):
    l = tr.step(tok[:, :-1], tok[:, 1:]).item()
  assert math.isfinite(l0) and l < l0


def test_kda_layer_training_step():
  torch.manual_seed(4)
  tr = Trainer(_cfg(attn="kda"))
  tok = torch.randint(0, 500, (2, 129))
  l0 = tr.step(tok[:, :-1], tok[:, 1:]).item()
  for _ in range(4):
    l = tr.step(tok[:, :-1], tok[:, 1:]).item()
  assert math.isfinite(l0) and l < l0


def test_indexer_backward_statement_matches_autograd():
  from nmoe_b200.ops.indexer import indexer_scores_backward, indexer_scores_ref
  torch.manual_seed(4)
  q = torch.randn(2, 24, 3, 8, requires_grad=True)
  k = torch.randn(2, 24, 8, requires_grad=True)
  w = torch.randn(2, 24, 3, requires_grad=True)
  g = torch.randn(2, 24, 24) * torch.tril(torch.ones(24, 24))
  (indexer_scores_ref(q, k, w, True).masked_fill(torch.triu(torch.ones(24, 24, dtype=torch.bool), 1), 0.0) * g).sum().backward()
  dq, dk, dw = indexer_scores_backward(q.detach(), k.detach(), w.detach(), g)
  for a, b in ((dq, q.grad), (dk, k.grad), (dw, w.grad)):
    assert torch.allclose(a, b, atol=1e-4, rtol=1e-4), (a - b).abs().max()
