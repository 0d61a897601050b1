"""Gated delta rule (KDA) chunk scan: the CUDA scan kernel against the loop statement, the differentiable chunked
operator against the token-by-token recurrence, and a layer-sized run at 4096 tokens."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
  return ((a.float() - b.float()).abs().max() / (b.float().abs().max() + 1e-9)).item()


@pytest.mark.parametrize("BH,n,Dk,Dv,reverse,with_g", [(3, 5, 192, 128, False, False), (2, 7, 64, 64, True, True),
                                                       (4, 3, 100, 192, False, True),
                                                       # enough (head, slice) pairs for 32- and 64-column slices per CTA
                                                       (40, 3, 128, 128, True, True), (80, 2, 128, 128, False, False)])
def test_scan_kernel_matches_loop(BH, n, Dk, Dv, reverse, with_g):
  from nmoe_b200.ops import kda as K
  torch.manual_seed(0)
  dev = "cuda"
  U = torch.randn(BH, n, 64, Dv, device=dev)
  P = torch.randn(BH, n, 64, Dk, device=dev) * 0.1
  K2 = torch.randn(BH, n, 64, Dk, device=dev) * 0.1
  dec = torch.rand(BH, n, Dk, device=dev) * 0.5 + 0.5
  G = torch.randn(BH, n, Dk, Dv, device=dev) * 0.1 if with_g else None
  W, H = K.scan(U, P, K2, dec, G, reverse)
  Wr, Hr = K._scan_loop(U, P, K2, dec, G, reverse)
  torch.cuda.synchronize()
  assert _rel(W, Wr) < 1e-4 and _rel(H, Hr) < 1e-4


def test_chunk_scan_forward_backward_matches_recurrence():
  from nmoe_b200.models.attention.kda import kda_recurrent
  from nmoe_b200.ops.kda import kda_chunk_scan
  torch.manual_seed(1)
  dev = "cuda"
  B, T, H, Dk, Dv = 2, 200, 2, 64, 64
  mk = lambda *s: torch.randn(*s, device=dev)
  q, k, v = mk(B, T, H, Dk).requires_grad_(), mk(B, T, H, Dk).requires_grad_(), mk(B, T, H, Dv).requires_grad_()
  g = (-torch.rand(B, T, H, Dk, device=dev) * 0.1).requires_grad_()
  beta = torch.rand(B, T, H, device=dev).requires_grad_()
  o = kda_chunk_scan(q, k, v, g, beta)
  go = torch.randn_like(o)
  got = torch.autograd.grad(o, (q, k, v, g, beta), go)
  o_ref = kda_recurrent(q, k, v, g, beta)
  want = torch.autograd.grad(o_ref, (q, k, v, g, beta), go)
  assert _rel(o, o_ref) < 1e-3
  for a, b in zip(got, want):
    assert _rel(a, b) < 5e-3


def test_kda_layer_at_4096_tokens():
  from nmoe_b200.config import Config
  from nmoe_b200.models.attention.kda import KDA
  from nmoe_b200.models.transformer import Transformer
  cfg = Config(vocab_size=512, eos_token_id=511, dim=512, n_layers=1, n_heads=4, inter_dim=256, n_dense_layers=1,
               q_lora_rank=128, kv_lora_rank=128, qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128,
               batch_size=2, seq_len=4096, max_position_embeddings=4096, attn="kda")
  torch.manual_seed(2)
  layer = KDA(cfg).cuda()
  layer.init_weights()
  rope = Transformer(cfg, dtype=torch.bfloat16, device=torch.device("cuda")).rope
  x = (torch.randn(2, 4096, cfg.dim, device="cuda") * 0.5).bfloat16().requires_grad_()
  y = layer(x, rope.cos[:4096], rope.sin[:4096])
  y.float().square().mean().backward()
  torch.cuda.synchronize()
  assert torch.isfinite(y.float()).all() and torch.isfinite(x.grad.float()).all() and x.grad.float().abs().max() > 0
