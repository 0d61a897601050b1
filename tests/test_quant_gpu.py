"""MXFP8 quantisation kernels (bit-exact vs the CPU emulation) and the block-scaled tcgen05 GEMM
(vs fp32 matmul of the dequantised operands)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
  return ((a.float() - b.float()).abs().max() / (b.float().abs().max() + 1e-6)).item()


def test_quant_mxfp8_bit_exact_vs_emulation():
  from nmoe_b200 import ops
  torch.manual_seed(0)
  x = (torch.randn(300, 512, device="cuda") * torch.logspace(-3, 2, 300, device="cuda").unsqueeze(1)).bfloat16()
  x[5, :64] = 0
  q, sf = ops.quant_mxfp8(x)
  qr, sfr = ops.quant_mxfp8(x.cpu())
  assert torch.equal(q.cpu(), qr)
  n = sfr.numel()
  from nmoe_b200.ref import quant as RQ
  got = RQ.sf_from_mma_layout(sf.cpu(), 384, 16)[:300]
  want = RQ.sf_from_mma_layout(sfr, 384, 16)[:300]
  assert torch.equal(got, want)
  d = ops.dequant_mxfp8(q, sf)
  assert _rel(d, x) < 0.07


def test_quant_mxfp4_bit_exact_vs_emulation():
  from nmoe_b200 import ops
  torch.manual_seed(1)
  x = (torch.randn(256, 256, device="cuda") * 3).bfloat16()
  q, sf = ops.quant_mxfp4(x)
  qr, sfr = ops.quant_mxfp4(x.cpu())
  assert torch.equal(q.cpu(), qr)
  assert torch.equal(sf.cpu(), sfr)


@pytest.mark.parametrize("M,N,K,bn", [(128, 128, 128, 128), (256, 256, 256, 256), (1000, 384, 512, 0), (300, 256, 2880, 0),
                                     (4096, 2816, 2048, 0)])
def test_gemm_mxfp8_vs_dequantised_matmul(M, N, K, bn):
  from nmoe_b200 import ops
  from nmoe_b200.ops import tc_gemm as G
  torch.manual_seed(2)
  a = torch.randn(M, K, device="cuda").bfloat16()
  b = (torch.randn(N, K, device="cuda") * 0.1).bfloat16()
  aq, asf = ops.quant_mxfp8(a)
  bq, bsf = ops.quant_mxfp8(b)
  c = ops.gemm_mxfp8(aq, asf, bq, bsf, bn=bn)
  torch.cuda.synchronize()
  G.check_status()
  ref = ops.dequant_mxfp8(aq, asf).float() @ ops.dequant_mxfp8(bq, bsf).float().t()
  assert _rel(c, ref) < 1e-2
  assert _rel(c, a.float() @ b.float().t()) < 8e-2


@pytest.mark.parametrize("M,N,K,bn", [(128, 128, 256, 128), (256, 256, 512, 256), (1000, 384, 1024, 0), (512, 256, 1408, 0),
                                     (4096, 2816, 2048, 0)])
def test_gemm_mxfp4_vs_dequantised_matmul(M, N, K, bn):
  """kind::mxf4nvf4 block-scaled GEMM vs fp32 matmul of the dequantised (E2M1 x E8M0) operands."""
  from nmoe_b200 import ops
  from nmoe_b200.ops import tc_gemm as G
  from nmoe_b200.ops.quant import gemm_mxfp4
  from nmoe_b200.ref import quant as RQ
  torch.manual_seed(3)
  a = torch.randn(M, K, device="cuda").bfloat16()
  b = (torch.randn(N, K, device="cuda") * 0.1).bfloat16()
  aq, asf = ops.quant_mxfp4(a)
  bq, bsf = ops.quant_mxfp4(b)
  c = gemm_mxfp4(aq, asf, bq, bsf, bn=bn)
  torch.cuda.synchronize()
  G.check_status()

  def deq(q, sf, rows):
    rp = (rows + 127) // 128 * 128
    s = RQ.sf_from_mma_layout(sf.cpu(), rp, ((K // 32) + 3) // 4 * 4)[:rows, :K // 32]
    return RQ.dequant_mxfp4(q.cpu(), s)

  ref = deq(aq, asf, M) @ deq(bq, bsf, N).t()
  assert _rel(c.cpu(), ref) < 1e-2
  assert _rel(c.cpu(), a.float().cpu() @ b.float().cpu().t()) < 0.35     # 4-bit operands


def test_moe_fp8_forward_close_to_bf16_and_backward_runs():
  from nmoe_b200.parallel.rdep import Rdep, moe_reference
  from nmoe_b200.ops.quant import ExpertWeightCache
  from nmoe_b200.ops import tc_gemm as G
  torch.manual_seed(3)
  dev = torch.device("cuda")
  T, H, F, E, K = 512, 256, 128, 8, 2
  rd = Rdep(H, E, K, T, device=dev, profile="fp8")
  try:
    x = (torch.randn(T, H, device=dev) * 0.5).bfloat16().requires_grad_()
    W13 = (torch.randn(E, 2 * F, H, device=dev) * 0.05).bfloat16().requires_grad_()
    W2 = (torch.randn(E, H, F, device=dev) * 0.05).bfloat16().requires_grad_()
    eid = torch.stack([torch.randperm(E, device=dev)[:K] for _ in range(T)]).int()
    gates = torch.rand(T, K, device=dev).requires_grad_()
    cache = ExpertWeightCache()
    out = rd.moe(x, gates, eid, W13, W2, False, cache.get(W13, W2))
    out.backward(torch.randn_like(out))
    torch.cuda.synchronize()
    G.check_status()
    ref = moe_reference(x.detach().float().cpu(), gates.detach().cpu(), eid.cpu().long(), W13.detach().float().cpu(),
                        W2.detach().float().cpu())
    assert (out.float().cpu() - ref).abs().max().item() < 8e-2 * ref.abs().max().item()   # two chained fp8 GEMMs
    assert torch.isfinite(x.grad).all() and torch.isfinite(W13.grad).all() and torch.isfinite(W2.grad).all()
    v0 = list(cache.ver)
    with torch.no_grad():
      W13.mul_(1.01)
    cache.get(W13, W2)
    assert cache.ver != v0
  finally:
    rd.close()


def test_moe_fp4_forward_close_to_bf16_and_backward_runs():
  """The 4-bit expert profile (E2M1 + E8M0/32 for tokens, activations and weights): quantising
  placement, both grouped GEMMs on kind::mxf4nvf4, fused return; bf16 straight-through backward."""
  from nmoe_b200.parallel.rdep import Rdep, moe_reference
  from nmoe_b200.ops.quant import ExpertWeightCache
  from nmoe_b200.ops import tc_gemm as G
  torch.manual_seed(4)
  dev = torch.device("cuda")
  T, H, F, E, K = 512, 256, 384, 8, 2           # F = 384: exercises the K % 256 == 128 tail of the down projection
  rd = Rdep(H, E, K, T, device=dev, profile="nvfp4")
  try:
    x = (torch.randn(T, H, device=dev) * 0.5).bfloat16().requires_grad_()
    W13 = (torch.randn(E, 2 * F, H, device=dev) * 0.05).bfloat16().requires_grad_()
    W2 = (torch.randn(E, H, F, device=dev) * 0.05).bfloat16().requires_grad_()
    eid = torch.stack([torch.randperm(E, device=dev)[:K] for _ in range(T)]).int()
    gates = torch.rand(T, K, device=dev).requires_grad_()
    cache = ExpertWeightCache("nvfp4")
    out = rd.moe(x, gates, eid, W13, W2, False, cache.get(W13, W2))
    out.backward(torch.randn_like(out))
    torch.cuda.synchronize()
    G.check_status()
    ref = moe_reference(x.detach().float().cpu(), gates.detach().cpu(), eid.cpu().long(), W13.detach().float().cpu(),
                        W2.detach().float().cpu())
    err = (out.float().cpu() - ref).abs().max().item() / ref.abs().max().item()
    cos = torch.nn.functional.cosine_similarity(out.float().cpu().flatten(), ref.flatten(), dim=0).item()
    assert err < 0.5 and cos > 0.95, (err, cos)      # two chained 4-bit GEMMs
    assert torch.isfinite(x.grad).all() and torch.isfinite(W13.grad).all() and torch.isfinite(W2.grad).all()
  finally:
    rd.close()


def test_moe_nvfp4_proper_is_closer_to_the_oracle_than_the_32_element_profile():
  """"nvfp4x16": E2M1 with one UE4M3 scale per 16 elements and an fp32 tensor scale (fixed for activations, from the
  maximum for weights, both left on the device) as an expert profile through the whole layer.  Finer blocks and a
  mantissa in the scale must give a smaller error than the E8M0-per-32 profile on the same data; backward is the bf16
  straight-through one and must match the bf16 profile's gradients closely."""
  from nmoe_b200.parallel.rdep import Rdep, moe_reference
  from nmoe_b200.ops.quant import ExpertWeightCache, ExpertWeightCacheNV16
  from nmoe_b200.ops import tc_gemm as G
  dev = torch.device("cuda")
  T, H, F, E, K = 512, 256, 384, 8, 2
  res = {}
  for profile in ("nvfp4", "nvfp4x16", "bf16"):
    torch.manual_seed(4)
    rd = Rdep(H, E, K, T, device=dev, profile=profile)
    try:
      x = (torch.randn(T, H, device=dev) * 0.5).bfloat16().requires_grad_()
      W13 = (torch.randn(E, 2 * F, H, device=dev) * 0.05).bfloat16().requires_grad_()
      W2 = (torch.randn(E, H, F, device=dev) * 0.05).bfloat16().requires_grad_()
      eid = torch.stack([torch.randperm(E, device=dev)[:K] for _ in range(T)]).int()
      gates = torch.rand(T, K, device=dev).requires_grad_()
      wq = None if profile == "bf16" else (ExpertWeightCacheNV16() if profile == "nvfp4x16" else ExpertWeightCache("nvfp4")).get(W13, W2)
      torch.manual_seed(9)
      out = rd.moe(x, gates, eid, W13, W2, False, wq)
      out.backward(torch.randn_like(out))
      torch.cuda.synchronize()
      G.check_status()
      ref = moe_reference(x.detach().float().cpu(), gates.detach().cpu(), eid.cpu().long(), W13.detach().float().cpu(),
                          W2.detach().float().cpu())
      err = ((out.float().cpu() - ref).pow(2).mean().sqrt() / ref.pow(2).mean().sqrt()).item()
      res[profile] = (err, x.grad.float().cpu(), W13.grad.float().cpu())
    finally:
      rd.close()
  assert res["nvfp4x16"][0] < 0.8 * res["nvfp4"][0], {k: v[0] for k, v in res.items()}
  assert res["nvfp4x16"][0] < 0.3, res["nvfp4x16"][0]          # two chained 4-bit GEMMs on contractions of 256 / 384
  for i in (1, 2):     # straight-through backward on the saved bf16 rows: the bf16 profile's gradients up to roundings
    a, b = res["nvfp4x16"][i], res["bf16"][i]
    assert (a - b).abs().max().item() <= 3e-2 * b.abs().max().item()


@pytest.mark.parametrize("M,N,K,bn", [(128, 128, 256, 128), (256, 256, 512, 256), (1000, 384, 1088, 0), (2048, 2816, 2048, 0)])
def test_gemm_nvfp4_vs_dequantised_matmul(M, N, K, bn):
  """True NVFP4 (16-element blocks, UE4M3 scales, fp32 tensor scale): quantiser bit-exact vs the emulation,
  GEMM vs fp32 matmul of the dequantised operands."""
  from nmoe_b200.ops import tc_gemm as G
  from nmoe_b200.ops.quant import gemm_nvfp4, quant_nvfp4
  from nmoe_b200.ref import quant as RQ
  torch.manual_seed(5)
  a = torch.randn(M, K, device="cuda").bfloat16()
  b = (torch.randn(N, K, device="cuda") * 0.1).bfloat16()
  aq, asf, ats = quant_nvfp4(a)
  bq, bsf, bts = quant_nvfp4(b)
  aq_r, asf_r, ats_r = quant_nvfp4(a.cpu())
  assert torch.equal(ats.cpu(), ats_r) and torch.equal(asf.cpu(), asf_r) and torch.equal(aq.cpu(), aq_r)
  c = gemm_nvfp4(aq, asf, ats, bq, bsf, bts, bn=bn)
  torch.cuda.synchronize()
  G.check_status()

  def deq(q, sf, ts, rows):
    rp = (rows + 127) // 128 * 128
    bs = RQ.sf_from_mma_layout(sf.cpu(), rp, ((K // 16) + 3) // 4 * 4)[:rows, :K // 16].contiguous().view(torch.float8_e4m3fn)
    return RQ.dequant_nvfp4(q.cpu(), bs, ts.cpu())

  ref = deq(aq, asf, ats, M) @ deq(bq, bsf, bts, N).t()
  assert _rel(c.cpu(), ref) < 1e-2
  assert _rel(c.cpu(), a.float().cpu() @ b.float().cpu().t()) < 0.3


@pytest.mark.parametrize("profile", ["fp8", "nvfp4"])
def test_blockscaled_moe_worst_case_routing(profile):
  """Every (token, slot) pair goes to expert 0 and the other experts are empty (the reference's worst-case
  test, tests/test_blockscaled_expert_worst_case.py:19-191): block-scaled path vs the fp32 MoE loop."""
  from nmoe_b200.parallel.rdep import Rdep, moe_reference
  from nmoe_b200.ops.quant import ExpertWeightCache
  from nmoe_b200.ops import tc_gemm as G
  torch.manual_seed(7)
  dev = torch.device("cuda")
  T, H, F, E, K = 384, 256, 256, 8, 1
  rd = Rdep(H, E, K, T, device=dev, profile=profile)
  try:
    x = (torch.randn(T, H, device=dev) * 0.5).bfloat16()
    W13 = (torch.randn(E, 2 * F, H, device=dev) * 0.05).bfloat16()
    W2 = (torch.randn(E, H, F, device=dev) * 0.05).bfloat16()
    eid = torch.zeros(T, K, dtype=torch.int32, device=dev)
    gates = torch.ones(T, K, device=dev)
    out = rd.moe(x, gates, eid, W13, W2, False, ExpertWeightCache(profile).get(W13, W2))
    torch.cuda.synchronize()
    G.check_status()
    ref = moe_reference(x.float().cpu(), gates.cpu(), eid.cpu().long(), W13.float().cpu(), W2.float().cpu())
    err = (out.float().cpu() - ref).abs().max().item() / ref.abs().max().item()
    assert torch.isfinite(out).all() and err < (8e-2 if profile == "fp8" else 0.5), err
  finally:
    rd.close()


@pytest.mark.parametrize("fp4", [False, True])
def test_fused_swiglu_quant_epilogue_matches_unfused(fp4):
  """Up/gate grouped GEMM with SwiGLU + quantise in its epilogue == GEMM -> bf16 H13 -> swiglu+quant kernel."""
  from nmoe_b200 import ops
  from nmoe_b200.ops import quant as Q
  from nmoe_b200.ops import tc_gemm as G
  torch.manual_seed(8)
  dev = torch.device("cuda")
  E, H, F, rows = 3, 256, 192, 512
  x = (torch.randn(rows, H, device=dev) * 0.5).bfloat16()
  W13 = (torch.randn(E, 2 * F, H, device=dev) * 0.1).bfloat16()
  quant = Q.quant_mxfp4 if fp4 else Q.quant_mxfp8
  xq, xsf = quant(x)
  wq, wsf = quant(W13.view(E * 2 * F, H))
  wq = wq.view(E, 2 * F, -1)
  tile_expert = torch.tensor([0, 0, 2, 1], dtype=torch.int32, device=dev)
  n_tiles = torch.tensor([4], dtype=torch.int32, device=dev)
  gg = Q.grouped_gemm_mxfp4 if fp4 else Q.grouped_gemm_mxfp8
  h13 = gg(xq, xsf, wq, wsf, tile_expert, n_tiles)
  aq_u, asf_u = (Q.swiglu_quant_mxfp4 if fp4 else Q.swiglu_quant_mxfp8)(h13, n_tiles)
  aq_f, asf_f = Q.grouped_gemm_swiglu_quant(xq, xsf, wq, wsf, tile_expert, n_tiles, fp4=fp4)
  torch.cuda.synchronize()
  G.check_status()
  assert torch.equal(aq_f, aq_u)
  n = Q.sf_bytes(rows, F)
  from nmoe_b200.ref import quant as RQ
  cols = ((F // 32) + 3) // 4 * 4
  su = RQ.sf_from_mma_layout(asf_u.cpu(), rows, cols)[:, :F // 32]
  sf_ = RQ.sf_from_mma_layout(asf_f.cpu(), rows, cols)[:, :F // 32]
  assert torch.equal(su, sf_)
  # the variant that also keeps H13 for the backward: same quantised activation, H13 bit-equal to the plain GEMM's
  aq_h, asf_h, h13_h = Q.grouped_gemm_swiglu_quant(xq, xsf, wq, wsf, tile_expert, n_tiles, fp4=fp4, want_h13=True)
  torch.cuda.synchronize()
  G.check_status()
  assert torch.equal(aq_h, aq_u) and torch.equal(h13_h, h13)
  assert torch.equal(RQ.sf_from_mma_layout(asf_h.cpu(), rows, cols)[:, :F // 32], su)


@pytest.mark.parametrize("profile", ["fp8", "nvfp4"])
def test_expert_adamw_refreshes_block_scaled_cache(profile):
  """The fused AdamW + quantise pass == flat AdamW followed by a fresh quantisation, and the optimizer
  drives it through the cache that the MoE layer registered on its parameters."""
  from nmoe_b200 import ops
  from nmoe_b200.config import Config
  from nmoe_b200.opt import ExpertAdamW
  from nmoe_b200.ops.quant import ExpertWeightCache
  torch.manual_seed(9)
  dev = torch.device("cuda")
  E, F, H = 4, 128, 256
  W13 = torch.nn.Parameter((torch.randn(E, 2 * F, H, device=dev) * 0.05).bfloat16())
  W2 = torch.nn.Parameter((torch.randn(E, H, F, device=dev) * 0.05).bfloat16())
  ref13, ref2 = W13.detach().clone(), W2.detach().clone()
  cache = ExpertWeightCache(profile)
  cache.get(W13, W2)
  cfg = Config()
  opt = ExpertAdamW([W13, W2], cfg)
  opt.begin_step(1e-2)
  g13, g2 = torch.randn_like(W13), torch.randn_like(W2)
  W13.grad, W2.grad = g13.clone(), g2.clone()
  opt.step()
  torch.cuda.synchronize()
  # oracle: plain flat AdamW on copies, then quantise
  for w, g in ((ref13, g13), (ref2, g2)):
    ops.adamw_flat_(w.view(-1), g.reshape(-1), torch.zeros_like(w).view(-1), torch.zeros_like(w).view(-1), lr=1e-2,
                    beta1=cfg.adam_beta1, beta2=cfg.adam_beta2_expert, eps=cfg.adam_eps, weight_decay=cfg.weight_decay, step=1)
  assert torch.equal(W13.detach(), ref13) and torch.equal(W2.detach(), ref2)
  fresh = ExpertWeightCache(profile)
  q13, s13, q2, s2 = fresh.get(W13, W2)
  c13, cs13, c2, cs2 = cache.get(W13, W2)
  assert cache.ver == [W13._version, W2._version]
  assert torch.equal(c13, q13) and torch.equal(c2, q2) and torch.equal(cs13, s13) and torch.equal(cs2, s2)
