"""Elementwise CUDA kernels vs the fp32 PyTorch oracle."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
  return ((a.float() - b.float()).abs().max() / (b.float().abs().max() + 1e-6)).item()


@pytest.mark.parametrize("M,H", [(37, 512), (1000, 2048), (64, 1536)])
def test_rmsnorm_fwd_bwd(M, H):
  from nmoe_b200 import ops
  from nmoe_b200.ref import ops as R
  torch.manual_seed(0)
  x = torch.randn(M, H, device="cuda").bfloat16().requires_grad_()
  w = (1 + 0.1 * torch.randn(H, device="cuda")).bfloat16().requires_grad_()
  y = ops.rmsnorm(x, w, 1e-5)
  g = torch.randn_like(y)
  y.backward(g)
  xf, wf = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
  yf = R.rmsnorm(xf, wf, 1e-5)
  yf.backward(g.float())
  assert _rel(y, yf) < 1e-2
  assert _rel(x.grad, xf.grad) < 2e-2
  assert _rel(w.grad, wf.grad) < 2e-2


def test_rope_fwd_bwd():
  from nmoe_b200 import ops
  from nmoe_b200.ref import ops as R
  torch.manual_seed(1)
  B, S, h, nope, rd = 2, 33, 4, 32, 16
  x = torch.randn(B, S, h, nope + rd, device="cuda").bfloat16().requires_grad_()
  ang = torch.rand(S, rd // 2, device="cuda") * 6.28
  cos, sin = ang.cos(), ang.sin()
  y = ops.rope(x, cos, sin, offset=nope)
  g = torch.randn_like(y)
  y.backward(g)
  xf = x.detach().float().requires_grad_()
  yf = torch.cat((xf[..., :nope], R.rope(xf[..., nope:], cos, sin)), -1)
  yf.backward(g.float())
  assert _rel(y, yf) < 1e-2
  assert _rel(x.grad, xf.grad) < 1e-2


def test_swiglu_fwd_bwd():
  from nmoe_b200 import ops
  from nmoe_b200.ref import ops as R
  torch.manual_seed(2)
  h = torch.randn(300, 2 * 704, device="cuda").bfloat16().requires_grad_()
  a = ops.swiglu(h)
  g = torch.randn_like(a)
  a.backward(g)
  hf = h.detach().float().requires_grad_()
  af = R.swiglu(hf[:, 0::2], hf[:, 1::2])
  af.backward(g.float())
  assert _rel(a, af) < 1e-2
  assert _rel(h.grad, hf.grad) < 2e-2


def test_embedding():
  from nmoe_b200 import ops
  torch.manual_seed(3)
  tab = torch.randn(1000, 256, device="cuda").bfloat16().requires_grad_()
  tok = torch.randint(0, 1000, (3, 50), device="cuda")
  y = ops.embedding(tok, tab, 10.667)
  ref = torch.nn.functional.embedding(tok, tab.detach().float()) * 10.667
  assert _rel(y, ref) < 1e-2
  y.sum().backward()
  cnt = torch.bincount(tok.view(-1), minlength=1000).float() * 10.667
  assert _rel(tab.grad.float().sum(-1), cnt * 256) < 1e-2


def test_adamw_flat():
  from nmoe_b200 import ops
  from nmoe_b200.ref import ops as R
  torch.manual_seed(4)
  n = 100003
  p = torch.randn(n, device="cuda").bfloat16()
  g = (torch.randn(n, device="cuda") * 0.1).bfloat16()
  m = torch.zeros_like(p)
  v = torch.zeros_like(p)
  pr, mr, vr = p.float().clone(), m.float().clone(), v.float().clone()
  for step in (1, 2, 3):
    ops.adamw_flat_(p, g, m, v, lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, step=step)
    R.adamw_step(pr, g.float(), mr, vr, lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, step=step)
    pr, mr, vr = pr.bfloat16().float(), mr.bfloat16().float(), vr.bfloat16().float()
  assert _rel(p, pr) < 2e-2


def test_newton_schulz_orthogonalises():
  from nmoe_b200.ops.muon import newton_schulz
  from nmoe_b200.ref import ops as R
  torch.manual_seed(5)
  x = torch.randn(3, 128, 256, device="cuda").bfloat16()
  y = newton_schulz(x)
  ref = R.newton_schulz(x.float().cpu())
  assert _rel(y.cpu(), ref) < 6e-2
  s = torch.linalg.svdvals(y.float())
  assert s.max() < 1.3 and s.min() > 0.5          # singular values pushed towards 1
  t = newton_schulz(torch.randn(256, 128, device="cuda").bfloat16())
  assert t.shape == (256, 128)


@pytest.mark.parametrize("M,H", [(300, 5120), (513, 7168)])
def test_rmsnorm_wide_rows_forward_backward(M, H):
  """Hidden sizes above 4096 (DeepSeek-V2 / V3 dims) take the two-pass backward."""
  from nmoe_b200 import ops
  from nmoe_b200.ref import ops as R
  torch.manual_seed(0)
  x = torch.randn(M, H, device="cuda").bfloat16().requires_grad_()
  w = (1 + 0.1 * torch.randn(H, device="cuda")).bfloat16().requires_grad_()
  y = ops.rmsnorm(x, w, 1e-6)
  g = torch.randn_like(y)
  y.backward(g)
  xf, wf = x.detach().float().cpu().requires_grad_(), w.detach().float().cpu().requires_grad_()
  yf = R.rmsnorm(xf, wf, 1e-6)
  yf.backward(g.float().cpu())
  rel = lambda a, b: ((a.float().cpu() - b).abs().max() / (b.abs().max() + 1e-6)).item()
  assert rel(y, yf.detach()) < 1e-2 and rel(x.grad, xf.grad) < 2e-2 and rel(w.grad, wf.grad) < 2e-2
