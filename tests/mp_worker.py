"""Multi-rank worker launched by test_multi_gpu.py through torch.distributed.run.

Checks on 2+ GPUs: RDEP MoE forward/backward against the fp32 oracle evaluated over the tokens of
ALL ranks, fused ZeRO-2 against the NCCL implementation, and a short lockstep training run."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from nmoe_b200 import runtime  # noqa: E402
from nmoe_b200.ops import tc_gemm as G  # noqa: E402


def rel(a, b):
  return ((a.float() - b.float()).abs().max() / (b.float().abs().max() + 1e-6)).item()


def close(a, ref, atol, rtol):
  """Largest per-element violation of |a - ref| <= atol + rtol * |ref| (<= 0 means every element passes)."""
  a, ref = a.float(), ref.float()
  return ((a - ref).abs() - (atol + rtol * ref.abs())).max().item()


def check_moe(rank, world, dev, profile="bf16", pipeline=False):
  from nmoe_b200.ops.quant import ExpertWeightCache
  from nmoe_b200.parallel.rdep import Rdep, moe_reference
  T, H, F, E, K = 384, 256, 128, 8, 2
  n_local = E // world
  g = torch.Generator().manual_seed(7)
  W13g = (torch.randn(E, 2 * F, H, generator=g) * 0.05).bfloat16()
  W2g = (torch.randn(E, H, F, generator=g) * 0.05).bfloat16()
  gr = torch.Generator().manual_seed(100 + rank)
  x = (torch.randn(T, H, generator=gr) * 0.5).bfloat16()
  eid = torch.stack([torch.randperm(E, generator=gr)[:K] for _ in range(T)]).int()
  gates = torch.rand(T, K, generator=gr)
  gout = torch.randn(T, H, generator=gr).bfloat16()
  rd = Rdep(H, E, K, T, device=dev, profile=profile)
  if pipeline:
    # the two halves of the tokens on two streams, each through its own peer buffers
    rd.make_halves()
    rd.pipe_min_tokens = 1
  xd = x.to(dev).requires_grad_()
  gd = gates.to(dev).requires_grad_()
  W13 = W13g[rank * n_local:(rank + 1) * n_local].to(dev).requires_grad_()
  W2 = W2g[rank * n_local:(rank + 1) * n_local].to(dev).requires_grad_()
  wq = ExpertWeightCache(profile).get(W13, W2) if profile != "bf16" else None
  for it in range(2):
    for t in (xd, gd, W13, W2):
      t.grad = None
    out = rd.moe(xd, gd, eid.to(dev), W13, W2, bool(it), wq)
    out.backward(gout.to(dev))
  torch.cuda.synchronize()
  G.check_status()
  # oracle over all ranks' tokens
  def gather(t):
    parts = [torch.empty_like(t.to(dev)) for _ in range(world)]
    dist.all_gather(parts, t.to(dev).contiguous())
    return torch.cat([p.cpu() for p in parts])
  xa, ea, ga, goa = gather(x), gather(eid), gather(gates), gather(gout)
  xf, gf = xa.float().requires_grad_(), ga.clone().requires_grad_()
  Wf, W2f = W13g.float().requires_grad_(), W2g.float().requires_grad_()
  ref = moe_reference(xf, gf, ea.long(), Wf, W2f)
  ref.backward(goa.float())
  sl = slice(rank * T, (rank + 1) * T)
  es = slice(rank * n_local, (rank + 1) * n_local)
  errs = {"out": rel(out.cpu(), ref[sl]), "dx": rel(xd.grad.cpu(), xf.grad[sl]), "dg": rel(gd.grad.cpu(), gf.grad[sl]),
          "dW13": rel(W13.grad.cpu(), Wf.grad[es]), "dW2": rel(W2.grad.cpu(), W2f.grad[es])}
  # forward, per element: |out - ref| <= atol_frac * max|ref| + rtol * |ref|.  bf16 is held to a few bf16 roundings
  # of the intermediates.  The block-scaled formats carry their element error into the sum (signed terms do not
  # average it away): two chained E4M3 GEMMs give a few percent of the output scale, E2M1 (two mantissa levels per
  # octave) several times that on contractions as short as this toy's 256 / 128; on the
  # reference's toy magnitudes these are its bars of 1e-2 / 5e-2 absolute (tests/test_rdep_accuracy.py:81-112).
  afrac, rtol, gtol = {"bf16": (6e-3, 1.6e-2, 3e-2), "fp8": (8e-2, 0.1, 8e-2), "nvfp4": (0.4, 0.5, 0.45)}[profile]
  errs["out_excess"] = close(out.cpu(), ref[sl], afrac * ref[sl].abs().max().item(), rtol)
  assert errs["out_excess"] <= 0, (profile, errs)
  assert all(v < gtol for k, v in errs.items() if k != "out_excess"), (profile, errs)
  dist.barrier()                                   # every peer's stores have landed
  assert rd.slab.check_guards() == [], rd.slab.check_guards()      # canaries (when NMOE_RDEP_GUARD is set)
  for h in (rd.halves or []):
    assert h.slab.check_guards() == [], h.slab.check_guards()
  dist.barrier()
  rd.close()
  return errs


def check_capacity_drop(rank, world, dev):
  """A receive buffer sized below the demand: rows beyond it are dropped, the status record says so (the host raises
  at its next check), nothing is written outside the regions, and the context stays usable."""
  from nmoe_b200.ops import _lib as L
  from nmoe_b200.parallel.rdep import Rdep
  T, H, F, E, K = 1024, 256, 128, 8, 2
  n_local = E // world
  rd = Rdep(H, E, K, T, device=dev, capacity_factor=0.25)     # room for a quarter of the balanced share
  g = torch.Generator().manual_seed(5 + rank)
  x = (torch.randn(T, H, generator=g) * 0.5).bfloat16().to(dev)
  eid = torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(T)]).int().to(dev)
  gates = torch.rand(T, K, generator=g).to(dev)
  W13 = (torch.randn(n_local, 2 * F, H, generator=g) * 0.05).bfloat16().to(dev)
  W2 = (torch.randn(n_local, H, F, generator=g) * 0.05).bfloat16().to(dev)
  out = rd.moe(x, gates, eid, W13, W2, False)
  torch.cuda.synchronize()
  dropped = False
  try:
    G.check_status()
  except L.NativeLibraryError as e:
    dropped = "code=" in str(e)
  flag = torch.tensor([int(dropped)], device=dev)
  dist.all_reduce(flag, op=dist.ReduceOp.MAX)
  assert int(flag.item()) == 1, "no rank reported dropped rows"
  assert torch.isfinite(out.float()).all()
  dist.barrier()
  assert rd.slab.check_guards() == []
  G.check_status()                     # the record was cleared by the raise
  dist.barrier()
  rd.close()
  return True


def check_zero2(rank, world, dev):
  from nmoe_b200.config import Config
  from nmoe_b200.parallel.zero2 import Zero2
  cfg = Config(dim=8, n_layers=1, n_heads=1)
  results = {}
  for impl in ("nccl", "fused"):
    cfg.zero2_impl = impl
    g = torch.Generator().manual_seed(3)
    params = [torch.nn.Parameter((torch.randn(n, generator=g)).bfloat16().to(dev)) for n in (1000, 4096, 77, 130000)]
    z = Zero2([{"name": "dense_decay", "params": params[:2], "lr": 1e-2, "weight_decay": 0.1},
               {"name": "router", "params": params[2:], "lr": 5e-3, "weight_decay": 0.0}], cfg)
    assert z.impl == impl
    for step in range(3):
      z.zero_grad()
      gg = torch.Generator().manual_seed(1000 * step + rank)
      for p in params:
        p.grad.copy_((torch.randn(p.numel(), generator=gg) * 0.1).bfloat16().view_as(p))
      z.step()
    torch.cuda.synchronize()
    G.check_status()
    results[impl] = torch.cat([p.detach().float().cpu().view(-1) for p in params])
    # every rank must hold identical parameters
    ref = results[impl].to(dev)
    other = ref.clone()
    dist.broadcast(other, src=0)
    assert torch.equal(ref, other), f"{impl}: ranks diverged"
  err = rel(results["fused"], results["nccl"])
  assert err < 1e-2, err
  return err


def check_zero2_overlap(rank, world, dev):
  """Bucketed ZeRO-2 stepped from backward hooks on a side stream == the same buckets stepped after backward,
  bit for bit (the update is elementwise and the ranks are summed in rank order either way)."""
  import os
  from nmoe_b200.config import Config
  from nmoe_b200.parallel.zero2 import Zero2
  cfg = Config(dim=8, n_layers=1, n_heads=1)
  cfg.zero2_impl = "fused"
  cfg.zero2_bucket_mb = 0.05                       # ~26k elements per bucket -> several buckets
  results = {}
  for overlap in (False, True):
    cfg.zero2_overlap = True
    g = torch.Generator().manual_seed(3)
    params = [torch.nn.Parameter((torch.randn(n, generator=g)).bfloat16().to(dev)) for n in (1000, 40960, 77, 130000, 512, 30000)]
    z = Zero2([{"name": "dense_decay", "params": params[:4], "lr": 1e-2, "weight_decay": 0.1},
               {"name": "router", "params": params[4:], "lr": 5e-3, "weight_decay": 0.0}], cfg)
    assert z.impl == "fused" and z.overlap and len(z.groups) >= 4, (z.impl, z.overlap, len(z.groups))
    gn = torch.zeros(1, device=dev)
    z.gradnorm_sq = gn
    for step in range(3):
      z.zero_grad()
      if not overlap:
        z._armed = False                           # same buckets, everything stepped by step()
      gg = torch.Generator().manual_seed(1000 * step + rank)
      loss = 0
      for p in params:
        c = (torch.randn(p.numel(), generator=gg) * 0.1).bfloat16().to(dev).view_as(p)
        loss = loss + (p * c).sum()
      loss.backward()
      if overlap:
        assert all(g_.launched for g_ in z.groups), [g_.launched for g_ in z.groups]
      z.step()
    torch.cuda.synchronize()
    G.check_status()
    results[overlap] = (torch.cat([p.detach().float().cpu().view(-1) for p in params]), float(gn.item()))
    sd = z.state_dict()
    z.load_state_dict(sd)
    dist.barrier()
  assert torch.equal(results[False][0], results[True][0])
  assert abs(results[False][1] - results[True][1]) <= 1e-3 * abs(results[False][1])
  return len(z.groups)


def check_train(rank, world, dev, overlap=False):
  import math
  from nmoe_b200.config import Config
  from nmoe_b200.train import Trainer
  cfg = Config(vocab_size=1024, eos_token_id=1023, dim=256, n_layers=3, n_heads=4, inter_dim=512, moe_inter_dim=128,
               n_routed_experts=8, n_activated_experts=2, n_shared_experts=1, n_dense_layers=1, q_lora_rank=96,
               kv_lora_rank=64, qk_nope_head_dim=32, qk_rope_head_dim=32, v_head_dim=32, batch_size=2 * world,
               seq_len=128, max_position_embeddings=256, warmup_steps=1, lr_dense=3e-3, lr_expert=3e-3, lr_router=3e-3)
  cfg.zero2_overlap = overlap
  cfg.zero2_bucket_mb = 0.25
  torch.manual_seed(11)                      # same dense init on every rank
  tr = Trainer(cfg, rank=rank, world=world, device=dev)
  assert tr.opt.dense.overlap == overlap
  g = torch.Generator().manual_seed(50 + rank)
  tok = torch.randint(0, 1000, (2, 129), generator=g)
  x, y = tok[:, :-1].contiguous(), tok[:, 1:].contiguous()
  losses = [tr.step(x, y).item() for _ in range(8)]
  G.check_status()
  assert math.isfinite(losses[0]) and losses[-1] < losses[0] - 0.05, losses
  # replicated parameters must stay identical across ranks
  flat = torch.cat([g_.flat_param.float() for g_ in tr.opt.dense.groups])
  other = flat.clone()
  dist.broadcast(other, src=0)
  assert torch.equal(flat, other)
  tr.model.rdep.close()
  return losses[0], losses[-1]


def main():
  rank, world, dev = runtime.init(0)
  out = {"moe": check_moe(rank, world, dev), "moe_fp8": check_moe(rank, world, dev, "fp8"),
         "moe_nvfp4": check_moe(rank, world, dev, "nvfp4"), "zero2": check_zero2(rank, world, dev),
         "moe_pipelined": check_moe(rank, world, dev, "bf16", pipeline=True),
         "moe_fp8_pipelined": check_moe(rank, world, dev, "fp8", pipeline=True),
         "zero2_overlap": check_zero2_overlap(rank, world, dev),
         "train": check_train(rank, world, dev), "train_overlap": check_train(rank, world, dev, overlap=True),
         "capacity_drop": check_capacity_drop(rank, world, dev)}
  dist.barrier()
  if rank == 0:
    print("MP_WORKER_OK", out, flush=True)
  runtime.finalize()


if __name__ == "__main__":
  main()
