"""tcgen05 GEMM family vs an fp32 PyTorch reference of the same contraction."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _close(c, ref, tol=2e-2):
  err = (c.float() - ref).abs().max().item()
  scale = ref.abs().max().item() + 1e-6
  assert err / scale < tol, f"rel err {err / scale:.4g} (abs {err:.4g}, scale {scale:.4g})"


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
@pytest.mark.parametrize("M,N,K,bn", [(128, 64, 64, 64), (256, 128, 128, 128), (384, 512, 320, 256),
                                      (1000, 264, 200, 0), (4096, 2048, 2048, 0)])
def test_dense_gemm(M, N, K, bn, a_mn, b_mn):
  from nmoe_b200.ops import tc_gemm as G
  torch.manual_seed(0)
  A = torch.randn(M, K, device="cuda")
  B = torch.randn(N, K, device="cuda")
  a = (A.t().contiguous() if a_mn else A).bfloat16()
  b = (B.t().contiguous() if b_mn else B).bfloat16()
  ref = (a.float().t() if a_mn else a.float()) @ (b.float() if b_mn else b.float().t())
  c = G.gemm(a, b, a_mn=a_mn, b_mn=b_mn, bn=bn)
  torch.cuda.synchronize()
  G.check_status()
  _close(c, ref)


def test_dense_gemm_fp32_accumulate():
  from nmoe_b200.ops import tc_gemm as G
  torch.manual_seed(1)
  a = torch.randn(512, 256, device="cuda").bfloat16()
  b = torch.randn(384, 256, device="cuda").bfloat16()
  out = torch.ones(512, 384, device="cuda")
  G.gemm(a, b, out=out, accumulate=True)
  G.gemm(a, b, out=out, accumulate=True)
  torch.cuda.synchronize()
  G.check_status()
  _close(out, 1 + 2 * (a.float() @ b.float().t()))


@pytest.mark.parametrize("b_mn", [False, True])
def test_grouped_gemm_rows(b_mn):
  from nmoe_b200.ops import tc_gemm as G
  torch.manual_seed(2)
  E, N, K = 5, 384, 256
  counts = [3, 0, 2, 1, 0]                       # 128-row tiles per expert (expert 1 and 4 empty)
  te = [e for e, c in enumerate(counts) for _ in range(c)]
  cap_tiles = 8
  a = torch.randn(cap_tiles * 128, K, device="cuda").bfloat16()
  w = torch.randn(E, N, K, device="cuda").bfloat16()
  wb = w.transpose(1, 2).contiguous() if b_mn else w
  tile_expert = torch.tensor(te + [-1] * (cap_tiles - len(te)), dtype=torch.int32, device="cuda")
  n_tiles = torch.tensor([len(te)], dtype=torch.int32, device="cuda")
  out = torch.full((cap_tiles * 128, N), 7.0, device="cuda", dtype=torch.bfloat16)
  G.grouped_gemm(a, wb, tile_expert, n_tiles, b_mn=b_mn, out=out)
  torch.cuda.synchronize()
  G.check_status()
  for i, e in enumerate(te):
    _close(out[i * 128:(i + 1) * 128], a[i * 128:(i + 1) * 128].float() @ w[e].float().t())
  assert (out[len(te) * 128:] == 7.0).all(), "rows past the valid tiles must not be written"


def test_grouped_wgrad():
  from nmoe_b200.ops import tc_gemm as G
  torch.manual_seed(3)
  E, Ma, Nb = 4, 320, 256
  rows = [256, 0, 128, 384]
  offs = torch.tensor([0] + list(torch.tensor(rows).cumsum(0)), dtype=torch.int32, device="cuda")
  R = sum(rows)
  a = torch.randn(R, Ma, device="cuda").bfloat16()
  b = torch.randn(R, Nb, device="cuda").bfloat16()
  out = G.grouped_wgrad(a, b, offs, E)
  torch.cuda.synchronize()
  G.check_status()
  o = offs.tolist()
  for e in range(E):
    ref = a[o[e]:o[e + 1]].float().t() @ b[o[e]:o[e + 1]].float()
    if rows[e] == 0:
      assert (out[e] == 0).all()
    else:
      _close(out[e], ref)


def test_linear_autograd():
  from nmoe_b200.ops import tc_gemm as G
  torch.manual_seed(4)
  x = torch.randn(4, 96, 256, device="cuda", dtype=torch.bfloat16, requires_grad=True)
  w = (torch.randn(512, 256, device="cuda") * 0.05).bfloat16().requires_grad_()
  y = G.linear(x, w)
  g = torch.randn_like(y)
  y.backward(g)
  xf, wf = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
  yf = torch.nn.functional.linear(xf, wf)
  yf.backward(g.float())
  torch.cuda.synchronize()
  G.check_status()
  _close(y, yf.detach())
  _close(x.grad, xf.grad)
  _close(w.grad, wf.grad)


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
@pytest.mark.parametrize("M,N,K", [(512, 256, 64), (1024, 512, 320), (1000, 776, 200), (4096, 2048, 2048)])
def test_pair_gemm(M, N, K, a_mn, b_mn):
  """Two-SM (cta_group::2) kernel, selected automatically for M >= 512 and N >= 256."""
  from nmoe_b200.ops import tc_gemm as G
  assert G.use_pair(M, N)
  torch.manual_seed(7)
  A = torch.randn(M, K, device="cuda")
  B = torch.randn(N, K, device="cuda")
  a = (A.t().contiguous() if a_mn else A).bfloat16()
  b = (B.t().contiguous() if b_mn else B).bfloat16()
  ref = (a.float().t() if a_mn else a.float()) @ (b.float() if b_mn else b.float().t())
  c = G.gemm(a, b, a_mn=a_mn, b_mn=b_mn)
  c1 = G.gemm(a, b, a_mn=a_mn, b_mn=b_mn, bn=256)        # one-SM kernel for comparison
  torch.cuda.synchronize()
  G.check_status()
  _close(c, ref)
  _close(c, c1.float(), tol=1e-2)


def test_pair_grouped_wgrad_and_fp32_accumulate():
  from nmoe_b200.ops import tc_gemm as G
  torch.manual_seed(8)
  E, Ma, Nb = 3, 640, 512
  rows = [256, 0, 384]
  offs = torch.tensor([0, 256, 256, 640], dtype=torch.int32, device="cuda")
  a = torch.randn(640, Ma, device="cuda").bfloat16()
  b = torch.randn(640, Nb, device="cuda").bfloat16()
  assert G.use_pair(Ma, Nb)
  out = G.grouped_wgrad(a, b, offs, E)
  acc = torch.ones(E, Ma, Nb, device="cuda")
  G.grouped_wgrad(a, b, offs, E, out=acc, accumulate=True)
  torch.cuda.synchronize()
  G.check_status()
  o = offs.tolist()
  for e in range(E):
    ref = a[o[e]:o[e + 1]].float().t() @ b[o[e]:o[e + 1]].float()
    if rows[e] == 0:
      assert (out[e] == 0).all() and (acc[e] == 1).all()
    else:
      _close(out[e], ref)
      _close(acc[e], 1 + ref)


@pytest.mark.parametrize("out_features", [4, 12, 20])
def test_linear_with_a_thin_output_has_a_right_backward(out_features):
  """A per-head scalar projection (4 outputs): in its backward the thin extent becomes a row stride (dy [M,4],
  dy^T), which TMA cannot address; the wrapper pads it.  Forward and both gradients against fp32."""
  from nmoe_b200 import ops
  torch.manual_seed(0)
  dev = torch.device("cuda")
  x = torch.randn(4096, 512, device=dev).bfloat16().requires_grad_(True)
  w = (torch.randn(out_features, 512, device=dev) * 0.05).bfloat16().requires_grad_(True)
  gy = torch.randn(4096, out_features, device=dev).bfloat16()
  y = ops.linear(x, w)
  y.backward(gy)
  xr, wr = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
  yr = xr @ wr.t()
  yr.backward(gy.float())
  for got, ref, name in ((y, yr, "y"), (x.grad, xr.grad, "dx"), (w.grad, wr.grad, "dw")):
    err = (got.float() - ref).abs().max().item()
    assert err <= 2e-2 * ref.abs().max().item() + 1e-3, (name, err, ref.abs().max().item())


@pytest.mark.parametrize("pair", [False, True])
def test_grouped_da_gemm_with_swiglu_backward_epilogue(pair, monkeypatch):
  """dA = dY W2 with the SwiGLU backward as its epilogue, against (a) the two-kernel form it replaces (same roundings:
  equal but for rare last-bit differences) and (b) an fp32 statement of the maths."""
  from nmoe_b200 import ops
  from nmoe_b200.ops import tc_gemm as G
  monkeypatch.setattr(G, "FUSED_SWIGLU_BWD", True)
  torch.manual_seed(5)
  dev = torch.device("cuda")
  E, H, F = 4, 512, 1408                         # F = 5.5 column tiles of 256: a ragged last tile
  counts = [4, 0, 2, 2] if pair else [3, 0, 2, 1]   # 128-row tiles per expert (256-aligned segments for CTA pairs)
  te = [e for e, c in enumerate(counts) for _ in range(c)]
  cap_tiles = 10
  M = cap_tiles * 128
  dy = (torch.randn(M, H, device=dev) * 0.5).bfloat16()
  w2 = (torch.randn(E, H, F, device=dev) * 0.05).bfloat16()
  h13 = torch.randn(M, 2 * F, device=dev).bfloat16()
  gate = torch.rand(M, device=dev) + 0.1
  tile_expert = torch.tensor(te + [-1] * (cap_tiles - len(te)), dtype=torch.int32, device=dev)
  n_tiles = torch.tensor([len(te)], dtype=torch.int32, device=dev)
  valid = len(te) * 128
  got = G.grouped_gemm_swiglu_bwd(dy, w2, tile_expert, n_tiles, h13, gate, align256=pair)
  assert got is not None
  dh, rowdot, a = got
  torch.cuda.synchronize()
  G.check_status()
  da = G.grouped_gemm(dy, w2, tile_expert, n_tiles, b_mn=True, align256=pair)
  dh2, rowdot2, a2 = ops.swiglu_bwd_fused(h13, da, gate, True, True, n_tiles)
  torch.cuda.synchronize()
  for x, y, name in ((dh, dh2, "dh13"), (a, a2, "a")):
    x, y = x[:valid].float(), y[:valid].float()
    same = (x == y).float().mean().item()
    assert same > 0.999, (name, same)
    assert ((x - y).abs() <= 2.0 ** -7 * y.abs() + 1e-30).all(), name          # never more than one bf16 step
  assert torch.allclose(rowdot[:valid], rowdot2[:valid], rtol=2e-3, atol=2e-2)
  # fp32 statement
  w_rows = torch.stack([w2[e] for e in te]).float()                              # [tiles, H, F]
  dA = torch.bmm(dy[:valid].float().view(len(te), 128, H), w_rows).view(valid, F)
  g, u = h13[:valid, 0::2].float(), h13[:valid, 1::2].float()
  s = torch.sigmoid(g)
  d = dA * gate[:valid].unsqueeze(-1)
  ref = torch.empty(valid, 2 * F, device=dev)
  ref[:, 0::2] = d * u * s * (1 + g * (1 - s))
  ref[:, 1::2] = d * g * s
  _close(dh[:valid], ref)
  _close(a[:valid], g * s * u * gate[:valid].unsqueeze(-1))
  rd = (g * s * u * dA).sum(-1)
  assert (rowdot[:valid] - rd).abs().max().item() <= 2e-2 * rd.abs().max().item()
