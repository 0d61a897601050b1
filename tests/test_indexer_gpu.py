"""Fused lightning-indexer score kernel against the fp32 statement of the op (values, mask, gradients)."""
import pytest
import torch

from nmoe_b200.ops.indexer import indexer_scores, indexer_scores_ref

pytestmark = pytest.mark.gpu


def _inputs(B, T, S, Hi, D, seed):
  g = torch.Generator(device="cuda").manual_seed(seed)
  q = torch.randn(B, T, Hi, D, device="cuda", generator=g).to(torch.bfloat16)
  k = torch.randn(B, S, D, device="cuda", generator=g).to(torch.bfloat16)
  w = torch.randn(B, T, Hi, device="cuda", generator=g).to(torch.bfloat16)
  return q, k, w


@pytest.mark.parametrize("B,T,S,Hi,D,causal", [
  (2, 512, 512, 4, 64, True),       # the module's default indexer
  (1, 300, 300, 16, 128, True),     # ragged tiles, two k-blocks
  (1, 256, 384, 64, 128, False),    # one query spans two 32-column chunks
  (1, 130, 200, 1, 64, False),      # one head
])
def test_indexer_scores_match_reference(B, T, S, Hi, D, causal):
  q, k, w = _inputs(B, T, S, Hi, D, 7)
  out = indexer_scores(q, k, w, causal)
  ref = indexer_scores_ref(q, k, w, causal)
  assert out.shape == ref.shape and out.dtype == torch.float32
  inf_ref = torch.isinf(ref)
  assert torch.equal(torch.isinf(out), inf_ref)
  a, b = out.masked_fill(inf_ref, 0.0), ref.masked_fill(inf_ref, 0.0)
  scale = b.abs().max().item()
  assert (a - b).abs().max().item() <= 2e-3 * scale + 1e-3, (a - b).abs().max().item()


def test_indexer_scores_gradients():
  q, k, w = _inputs(2, 192, 192, 4, 64, 11)
  leaves = [t.clone().requires_grad_(True) for t in (q, k, w)]
  refs = [t.clone().float().requires_grad_(True) for t in (q, k, w)]
  g = torch.randn(2, 192, 192, device="cuda")
  mask = torch.tril(torch.ones(192, 192, dtype=torch.bool, device="cuda"))
  (indexer_scores(*leaves, True).masked_fill(~mask, 0.0) * g).sum().backward()
  (indexer_scores_ref(*refs, True).masked_fill(~mask, 0.0) * g).sum().backward()
  for a, b in zip(leaves, refs):
    err = (a.grad.float() - b.grad).abs().max().item()
    assert err <= 2e-2 * b.grad.abs().max().item() + 1e-3, err


def test_dsa_block_runs_fused_indexer():
  from nmoe_b200.models.attention import dsa

  torch.manual_seed(3)
  q, k, w = _inputs(1, 256, 256, 4, 64, 5)
  vals, idx = dsa.lightning_indexer(q, k, w, 32)
  ref = indexer_scores_ref(q, k, w, True)
  rv, _ = ref.topk(32, dim=-1)
  fin = ~torch.isinf(rv)
  assert torch.equal(torch.isinf(vals), ~fin)
  assert (vals[fin] - rv[fin]).abs().max().item() <= 2e-3 * rv[fin].abs().max().item() + 1e-3
  t = torch.arange(256, device="cuda").view(1, 256, 1)
  assert ((idx <= t) | ~fin).all()
