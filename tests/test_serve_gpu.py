"""Serving kernels and engine on the GPU vs the fp32 statements of the same maths."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
  return ((a.float() - b.float()).abs().max() / (b.float().abs().max() + 1e-6)).item()


@pytest.mark.parametrize("D,Hq,Hkv,window,use_sinks", [(64, 8, 2, 0, True), (64, 64, 8, 128, True), (128, 16, 16, 0, False),
                                                        (128, 32, 4, 40, True)])
def test_paged_decode_and_kv_store_vs_oracle(D, Hq, Hkv, window, use_sinks):
  from nmoe_b200.serve import ops as S
  torch.manual_seed(0)
  dev = torch.device("cuda")
  B, bs, nb = 5, 16, 64
  ctx = torch.tensor([1, 17, 100, 250, 33], dtype=torch.int32)
  max_blocks = int((ctx.max() + bs - 1) // bs)
  perm = torch.randperm(nb)
  tables = torch.zeros(B, max_blocks, dtype=torch.int32)
  used = 0
  for b in range(B):
    n = int((ctx[b] + bs - 1) // bs)
    tables[b, :n] = perm[used:used + n].int()
    used += n
  k_cache = torch.zeros(nb, bs, Hkv, D, device=dev, dtype=torch.bfloat16)
  v_cache = torch.zeros_like(k_cache)
  # fill the cache through the scatter kernel, token by token order shuffled, some rows skipped
  for b in range(B):
    n = int(ctx[b])
    k = torch.randn(n + 2, Hkv, D, device=dev).bfloat16()
    v = torch.randn(n + 2, Hkv, D, device=dev).bfloat16()
    pos = torch.arange(n)
    slots = torch.full((n + 2,), -1, dtype=torch.int32)
    slots[:n] = tables[b, pos // bs] * bs + (pos % bs).int()
    S.kv_store(k, v, k_cache, v_cache, slots.to(dev))
    kc = k_cache.view(-1, Hkv, D)[slots[:n].long().to(dev)]
    assert torch.equal(kc, k[:n])
  q = torch.randn(B, Hq, D, device=dev).bfloat16()
  sinks = torch.randn(Hq, device=dev) if use_sinks else None
  out = S.paged_decode(q, k_cache, v_cache, tables.to(dev), ctx.to(dev), sinks, D ** -0.5, window)
  torch.cuda.synchronize()
  ref = S.paged_decode_reference(q.cpu(), k_cache.cpu(), v_cache.cpu(), tables, ctx, sinks.cpu() if use_sinks else None,
                                 D ** -0.5, window)
  assert _rel(out.cpu(), ref) < 2e-2


def test_engine_gpu_logits_track_fp32_model_and_prefix_cache_is_consistent():
  from nmoe_b200.serve import Engine, ServeConfig, Transformer
  from nmoe_b200.ops import tc_gemm as G
  torch.manual_seed(0)
  cfg = ServeConfig(num_hidden_layers=3, num_experts=8, experts_per_token=2, vocab_size=512, hidden_size=256,
                    intermediate_size=160, head_dim=64, num_attention_heads=8, num_key_value_heads=2, sliding_window=16,
                    initial_context_length=128, rope_scaling_factor=1.0, probe_layer=2, judge_layer=3)
  dev = torch.device("cuda")
  mg = Transformer(cfg, dtype=torch.bfloat16, device=dev, max_tokens=512)
  mg.init_weights(std=0.05)
  mc = Transformer(cfg, dtype=torch.float32)
  mc.load_state_dict({k: v.float().cpu() for k, v in mg.state_dict().items()})
  shared = list(range(40, 72))
  prompts = [shared + [5, 6, 7], shared + [9], [100, 101, 102, 103, 104]]
  try:
    eg = Engine(mg, max_seq_len=96, max_batch=4)
    ec = Engine(mc, max_seq_len=96, max_batch=4)
    for p in prompts:
      eg.add(p, 4); ec.add(p, 4)
    lg, ids_g = eg.step()
    lc, ids_c = ec.step()
    torch.cuda.synchronize()
    G.check_status()
    assert torch.isfinite(lg).all()
    cos = torch.nn.functional.cosine_similarity(lg.cpu().flatten(), lc.flatten(), dim=0).item()
    assert cos > 0.98, cos
    # advance both with the fp32 model's tokens: decode path (paged attention) must keep tracking
    for _ in range(3):
      nxt = lc.argmax(-1).tolist()
      for sg, sc, t in zip(ids_g, ids_c, nxt):
        eg.update(sg, t); ec.update(sc, t)
      lg, ids_g = eg.step()
      lc, ids_c = ec.step()
      cos = torch.nn.functional.cosine_similarity(lg.cpu().flatten(), lc.flatten(), dim=0).item()
      assert cos > 0.95, cos        # bf16 + MXFP8 experts vs fp32, a few near-tied routing decisions flip
    # a fourth request sharing the (now cached) prefix: its prefill must agree with the fp32 engine
    eg.add(shared + [11, 12], 2); ec.add(shared + [11, 12], 2)
    for e in (eg, ec):
      for s in list(e.running):
        e.update(s.seq_id, 0, finished=True)
    lg, _ = eg.step()
    lc, _ = ec.step()
    assert eg.steps["cached_tokens"] >= 32 and ec.steps["cached_tokens"] >= 32
    cos = torch.nn.functional.cosine_similarity(lg.cpu().flatten(), lc.flatten(), dim=0).item()
    assert cos > 0.95, cos
    G.check_status()
  finally:
    if mg.rdep is not None:
      mg.rdep.close()
