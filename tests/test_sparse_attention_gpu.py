"""Token-sparse attention on the tcgen05 kernels: packed bit masks (top-k select, block lists, fixed positions,
bit transpose) and the masked forward / backward against the fp32 eager statement; DSA and NSA layers on that path."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
  return ((a.float() - b.float()).abs().max() / (b.float().abs().max() + 1e-6)).item()


@pytest.mark.parametrize("B,S,k", [(2, 300, 17), (1, 1024, 256), (1, 129, 500)])
def test_topk_mask_matches_sorting(B, S, k):
  from nmoe_b200.ops.attention import SparseMask
  torch.manual_seed(0)
  scores = torch.randn(B, S, S, device="cuda")
  scores[:, :, 5] = float("-inf")                               # a key that must never be chosen
  m = SparseMask.from_topk_scores(scores, k)
  got = m.to_bool()
  causal = torch.tril(torch.ones(S, S, dtype=torch.bool, device="cuda"))
  s = scores.masked_fill(~causal, float("-inf"))
  vals, idx = s.topk(min(k, S), dim=-1)
  want = torch.zeros(B, S, S, dtype=torch.bool, device="cuda").scatter_(2, idx, vals > float("-inf"))
  assert torch.equal(got, want)
  # transpose
  sh = torch.arange(32, device="cuda", dtype=torch.int64)
  wt = ((m.bits_t.to(torch.int64) & 0xFFFFFFFF).unsqueeze(-1) >> sh & 1).bool().view(B, S, -1)[..., :S]
  assert torch.equal(wt, want.transpose(1, 2))


def test_topk_mask_admits_ties_in_key_order():
  from nmoe_b200.ops.attention import SparseMask
  S = 96
  scores = torch.zeros(1, S, S, device="cuda")                   # every score equal: the k lowest key indices win
  got = SparseMask.from_topk_scores(scores, 10).to_bool()[0]
  for q in (0, 3, 9, 10, 50, 95):
    assert got[q].nonzero().flatten().tolist() == list(range(min(q + 1, 10)))


def test_block_and_position_masks():
  from nmoe_b200.ops.attention import SparseMask
  B, S, bs = 2, 200, 16
  torch.manual_seed(1)
  blocks = torch.randint(-1, (S + bs - 1) // bs, (B, S, 5), device="cuda", dtype=torch.int32)
  got = SparseMask.from_blocks(blocks, bs, S).to_bool()
  want = SparseMask.from_blocks(blocks.cpu(), bs, S).to_bool()
  assert torch.equal(got.cpu(), want)
  pos = torch.tensor([0, 31, 32, 63, 64, 199, 500, -3], device="cuda")
  got = SparseMask.from_positions(pos, B, S).to_bool()
  assert got[1, 17].nonzero().flatten().tolist() == [0, 31, 32, 63, 64, 199]


@pytest.mark.parametrize("B,S,Hq,Hkv,Dqk,Dv,window,keep", [
  (2, 300, 2, 2, 192, 128, 0, 0.3),
  (1, 512, 4, 2, 128, 128, 0, 0.1),
  (1, 330, 4, 1, 64, 64, 100, 0.5),
])
def test_masked_attention_forward_backward(B, S, Hq, Hkv, Dqk, Dv, window, keep):
  from nmoe_b200.models.attention.common import masked_attention
  from nmoe_b200.ops import tc_gemm as G
  from nmoe_b200.ops.attention import SparseMask, attention
  torch.manual_seed(2)
  q = torch.randn(B, S, Hq, Dqk, device="cuda").bfloat16().requires_grad_()
  k = torch.randn(B, S, Hkv, Dqk, device="cuda").bfloat16().requires_grad_()
  v = torch.randn(B, S, Hkv, Dv, device="cuda").bfloat16().requires_grad_()
  go = torch.randn(B, S, Hq, Dv, device="cuda").bfloat16()
  scores = torch.rand(B, S, S, device="cuda")
  scores = scores.masked_fill(scores > keep, float("-inf"))       # a random subset of keys per query (some rows empty)
  mask = SparseMask.from_topk_scores(scores, S)
  scale = Dqk ** -0.5
  o = attention(q, k, v, scale, window=window, mask=mask)
  o.backward(go)
  torch.cuda.synchronize()
  G.check_status()
  qf, kf, vf = (t.detach().float().requires_grad_() for t in (q, k, v))
  i = torch.arange(S, device="cuda").unsqueeze(-1); j = torch.arange(S, device="cuda").unsqueeze(0)
  allowed = mask.to_bool() & (j <= i)
  if window > 0:
    allowed = allowed & (j > i - window)
  ref = masked_attention(qf, kf, vf, allowed.unsqueeze(1), scale)
  ref.backward(go.float())
  assert _rel(o, ref) < 2e-2
  assert _rel(q.grad, qf.grad) < 3e-2 and _rel(k.grad, kf.grad) < 3e-2 and _rel(v.grad, vf.grad) < 3e-2


def _cfg(**kw):
  from nmoe_b200.config import Config
  base = dict(vocab_size=512, eos_token_id=511, dim=256, n_layers=1, n_heads=2, inter_dim=256, n_dense_layers=1,
              q_lora_rank=64, kv_lora_rank=64, qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128, batch_size=2,
              seq_len=256, max_position_embeddings=4096)
  base.update(kw)
  return Config(**base)


def test_dsa_sparse_layer_matches_eager_statement():
  from nmoe_b200.models.attention.dsa import DSA
  from nmoe_b200.ops import tc_gemm as G
  torch.manual_seed(3)
  cfg = _cfg(attn="dsa", attn_dsa={"top_k": 48, "n_idx_heads": 4, "idx_dim": 64})
  layer = DSA(cfg).cuda()
  layer.init_weights()
  T = 256
  from nmoe_b200.models.transformer import Transformer
  model_rope = Transformer(cfg, dtype=torch.bfloat16, device=torch.device("cuda")).rope
  cos, sin = model_rope.cos[:T], model_rope.sin[:T]
  x = (torch.randn(2, T, cfg.dim, device="cuda") * 0.5).bfloat16().requires_grad_()
  y = layer(x, cos, sin)
  y.float().square().mean().backward()
  gx = x.grad.clone()
  loss = layer.indexer_alignment_loss()
  torch.cuda.synchronize()
  G.check_status()
  assert torch.isfinite(loss)
  # the same layer through its eager branch (fp32 weights, [T, T] masks)
  ref = DSA(cfg, dtype=torch.float32).cuda()
  ref.load_state_dict({k_: v_.float() for k_, v_ in layer.state_dict().items()})
  xr = x.detach().float().requires_grad_()
  yr = ref(xr, cos.float(), sin.float())
  yr.square().mean().backward()
  # a near-tie in the indexer scores may pick a different key in bf16 than in fp32
  assert _rel(y, yr) < 8e-2 and _rel(gx, xr.grad) < 0.15


def test_nsa_selection_branch_on_the_masked_kernel():
  from nmoe_b200.models.attention.nsa import NSA
  from nmoe_b200.ops import tc_gemm as G
  torch.manual_seed(4)
  cfg = _cfg(attn="nsa", n_heads=4, qk_nope_head_dim=64, qk_rope_head_dim=64, v_head_dim=128,
             attn_nsa={"cmp_len": 32, "cmp_stride": 16, "slc_block": 64, "topk_blocks": 4, "kv_heads": 2})
  nsa = NSA(cfg).cuda()
  B, T, H, KV, D = 2, 512, 4, 2, 128
  q = torch.randn(B, T, H, D, device="cuda").bfloat16()
  k = torch.randn(B, T, KV, D, device="cuda").bfloat16()
  v = torch.randn(B, T, KV, D, device="cuda").bfloat16()
  blocks = nsa.select_blocks(torch.rand(B, T, KV, T // 64, device="cuda"), T)
  got = nsa.slc_attention(q, k, v, blocks)
  torch.cuda.synchronize()
  G.check_status()
  want = nsa.slc_attention(q.float().cpu(), k.float().cpu(), v.float().cpu(), blocks.cpu())
  assert _rel(got.cpu(), want) < 2e-2


def test_dsa_at_4096_tokens_builds_no_per_head_quadratic_tensor():
  from nmoe_b200.models.attention.dsa import DSA
  from nmoe_b200.models.transformer import Transformer
  from nmoe_b200.ops import tc_gemm as G
  cfg = _cfg(attn="dsa", n_heads=16, dim=1024, attn_dsa={"top_k": 1024, "n_idx_heads": 4, "idx_dim": 64}, seq_len=4096)
  layer = DSA(cfg).cuda()
  layer.init_weights()
  rope = Transformer(_cfg(seq_len=4096), dtype=torch.bfloat16, device=torch.device("cuda")).rope
  B, T = 2, 4096
  x = (torch.randn(B, T, cfg.dim, device="cuda") * 0.5).bfloat16().requires_grad_()
  torch.cuda.synchronize()
  torch.cuda.reset_peak_memory_stats()
  base = torch.cuda.memory_allocated()
  y = layer(x, rope.cos[:T], rope.sin[:T])
  y.float().mean().backward()
  torch.cuda.synchronize()
  G.check_status()
  peak = torch.cuda.max_memory_allocated() - base
  # one [B, H, T, T] fp32 tensor alone would be 2 * 16 * 4096^2 * 4 B = 2 GiB; forward + backward of the whole layer
  # (including the head-summed indexer scores [B, T, T], 128 MiB) stay below that
  assert peak < 1.5 * 2 ** 30, peak / 2 ** 30
  assert torch.isfinite(x.grad.float()).all()


@pytest.mark.parametrize("D,T,mode", [(128, 1024, "random"), (64, 1000, "random"), (128, 4096, "random"), (128, 512, "negative")])
def test_nsa_compressed_attention_kernels_vs_statement(D, T, mode):
  """Forward (output + selection-block scores) and the three gradients of the compressed branch against the PyTorch
  statement in fp32.  "negative" makes every score negative and large, so the floors of the maximum (0) and of the
  denominator (1e-6) are what decides the result."""
  from nmoe_b200.ops import nsa as N
  from nmoe_b200.ops import tc_gemm as G
  torch.manual_seed(0)
  dev = torch.device("cuda")
  B, KV, l, d, blk = 2, 2, 32, 16, 64
  Tc = (T - l) // d + 1
  q = torch.randn(B, T, KV, D, device=dev)
  kc = torch.randn(B, Tc, KV, D, device=dev)
  vc = torch.randn(B, Tc, KV, D, device=dev)
  scale = D ** -0.5
  if mode == "negative":
    q, kc, scale = q.abs(), -kc.abs() - 0.2, 0.25
  q, kc, vc = (x.bfloat16().requires_grad_(True) for x in (q, kc, vc))
  assert N.kernel_ok(q, kc, blk)
  out, scores = N.cmp_attention(q, kc, vc, cmp_len=l, cmp_stride=d, slc_block=blk, scale=scale)
  go = torch.randn_like(out)
  out.backward(go)
  torch.cuda.synchronize()
  G.check_status()
  qf, kf, vf = (x.detach().float().requires_grad_(True) for x in (q, kc, vc))
  ro, rs = N.cmp_attention_reference(qf, kf, vf, cmp_len=l, cmp_stride=d, slc_block=blk, scale=scale)
  ro.backward(go.float())
  assert not scores.requires_grad and scores.shape == rs.shape
  def close(a, b, name, tol=2e-2):
    err = (a.float() - b.float()).abs().max().item()
    ref = b.float().abs().max().item()
    assert err <= tol * ref + 1e-6, (name, err, ref)
  close(out, ro, "out")
  close(scores, rs, "scores", 5e-3)
  assert (scores[:, :l - 1] == 0).all() and (out[:, :l - 1] == 0).all()       # nothing visible before the first block ends
  close(q.grad, qf.grad, "dq")
  close(kc.grad, kf.grad, "dkc")
  close(vc.grad, vf.grad, "dvc")
  if mode == "negative":
    assert float(ro.abs().max()) > 0            # the case is not degenerate: some rows sit on the denominator's floor
    den = torch.exp((torch.einsum("bthd,bchd->bhtc", qf, kf) * scale)[..., -1, :]).sum(-1)
    assert (den < 1e-6).any()
