"""tcgen05 attention forward vs the fp32 eager oracle: MLA dims, sliding window, sinks, GQA, ragged S."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
  return ((a.float() - b.float()).abs().max() / (b.float().abs().max() + 1e-6)).item()


@pytest.mark.parametrize("B,S,Hq,Hkv,Dqk,Dv,window,use_sinks", [
  (2, 256, 4, 4, 192, 128, 0, False),
  (1, 1024, 2, 2, 192, 128, 0, False),
  (2, 384, 4, 2, 128, 128, 128, True),
  (1, 512, 4, 4, 128, 128, 100, False),
  (1, 300, 2, 1, 64, 64, 0, True),
  (1, 640, 2, 2, 64, 64, 37, True),
])
def test_attention_forward_and_lse(B, S, Hq, Hkv, Dqk, Dv, window, use_sinks):
  from nmoe_b200.ops.attention import attention_forward
  from nmoe_b200.ops import tc_gemm as G
  from nmoe_b200.ref import ops as R
  torch.manual_seed(0)
  q = torch.randn(B, S, Hq, Dqk, device="cuda").bfloat16()
  k = torch.randn(B, S, Hkv, Dqk, device="cuda").bfloat16()
  v = torch.randn(B, S, Hkv, Dv, device="cuda").bfloat16()
  sinks = (torch.randn(Hq, device="cuda") * 2).bfloat16() if use_sinks else None
  scale = Dqk ** -0.5
  o, lse = attention_forward(q, k, v, scale, window, sinks)
  torch.cuda.synchronize()
  G.check_status()
  ref = R.attention(q.float().cpu(), k.float().cpu(), v.float().cpu(), scale, window=window,
                    sinks=sinks.float().cpu() if sinks is not None else None)
  assert _rel(o.cpu(), ref) < 2e-2
  # lse against eager
  kk = k.float().cpu().repeat_interleave(Hq // Hkv, dim=2)
  s = torch.einsum("bihd,bjhd->bhij", q.float().cpu(), kk) * scale
  i = torch.arange(S).unsqueeze(-1); j = torch.arange(S).unsqueeze(0)
  mask = j <= i
  if window > 0:
    mask &= j > i - window
  s = s.masked_fill(~mask, float("-inf"))
  if sinks is not None:
    s = torch.cat((s, sinks.float().cpu().view(1, Hq, 1, 1).expand(B, Hq, S, 1)), -1)
  assert torch.allclose(lse.cpu(), torch.logsumexp(s, -1), atol=2e-2, rtol=1e-3)


@pytest.mark.parametrize("B,S,Hq,Hkv,Dqk,Dv,window,use_sinks", [
  (1, 256, 2, 2, 192, 128, 0, False),
  (2, 640, 2, 2, 192, 128, 0, False),
  (1, 256, 2, 2, 128, 128, 64, True),
  (1, 448, 4, 2, 128, 128, 0, False),
  (1, 300, 4, 1, 64, 64, 0, True),
  (2, 330, 2, 2, 64, 64, 100, False),
])
def test_attention_backward_kernels(B, S, Hq, Hkv, Dqk, Dv, window, use_sinks):
  """dQ / dK / dV (and the sink gradient) of the tcgen05 backward vs autograd through the fp32 oracle."""
  from nmoe_b200.ops.attention import attention
  from nmoe_b200.ops import tc_gemm as G
  from nmoe_b200.ref import ops as R
  torch.manual_seed(1)
  q = torch.randn(B, S, Hq, Dqk, device="cuda").bfloat16().requires_grad_()
  k = torch.randn(B, S, Hkv, Dqk, device="cuda").bfloat16().requires_grad_()
  v = torch.randn(B, S, Hkv, Dv, device="cuda").bfloat16().requires_grad_()
  sinks = torch.randn(Hq, device="cuda").bfloat16().requires_grad_() if use_sinks else None
  o = attention(q, k, v, Dqk ** -0.5, window=window, sinks=sinks)
  g = torch.randn_like(o)
  o.backward(g)
  torch.cuda.synchronize()
  G.check_status()
  qf, kf, vf = (t.detach().float().cpu().requires_grad_() for t in (q, k, v))
  sf = sinks.detach().float().cpu().requires_grad_() if use_sinks else None
  of = R.attention(qf, kf, vf, Dqk ** -0.5, window=window, sinks=sf)
  of.backward(g.float().cpu())
  assert _rel(o.cpu(), of.detach()) < 2e-2
  for name, a, b in (("dq", q.grad, qf.grad), ("dk", k.grad, kf.grad), ("dv", v.grad, vf.grad)):
    assert torch.isfinite(a).all(), name
    assert _rel(a.cpu(), b) < 3e-2, name
  if use_sinks:
    assert _rel(sinks.grad.cpu(), sf.grad) < 5e-2


def test_mla_attention_split_sources_matches_materialised():
  from nmoe_b200.ops.attention import attention, mla_attention
  torch.manual_seed(2)
  B, S, H, nope, rope, vd = 2, 384, 4, 128, 64, 128
  q = torch.randn(B, S, H, nope + rope, device="cuda").bfloat16().requires_grad_()
  kv = torch.randn(B, S, H, nope + vd, device="cuda").bfloat16().requires_grad_()
  pe = torch.randn(B, S, 1, rope, device="cuda").bfloat16().requires_grad_()
  o = mla_attention(q, kv, pe, 192 ** -0.5, nope, vd)
  g = torch.randn_like(o)
  o.backward(g)
  q2, kv2, pe2 = (t.detach().clone().requires_grad_() for t in (q, kv, pe))
  k = torch.cat((kv2[..., :nope], pe2.expand(B, S, H, rope)), -1)
  o2 = attention(q2, k, kv2[..., nope:].contiguous(), 192 ** -0.5)
  o2.backward(g)
  assert torch.equal(o, o2)
  for a, b in ((q.grad, q2.grad), (kv.grad, kv2.grad), (pe.grad, pe2.grad)):
    assert _rel(a, b) < 2e-2
  # and against autograd through the fp32 oracle
  from nmoe_b200.ref import ops as R
  qf, kvf, pef = (t.detach().float().cpu().requires_grad_() for t in (q, kv, pe))
  kf = torch.cat((kvf[..., :nope], pef.expand(B, S, H, rope)), -1)
  of = R.attention(qf, kf, kvf[..., nope:], 192 ** -0.5)
  of.backward(g.float().cpu())
  for a, b in ((q.grad, qf.grad), (kv.grad, kvf.grad), (pe.grad, pef.grad)):
    assert _rel(a.cpu(), b) < 3e-2
