"""Routed-expert layer, this framework against the unmodified reference, same process, same inputs.

  python benchmarks/moe_layer.py [--shape moonlight|dsv3] [--tokens 16384] [--dtype bf16|fp8|nvfp4]
                                 [--routing uniform|zipf] [--impl both|ours|reference] [--backward]
  torchrun --nnodes 1 --nproc-per-node N --master-addr 127.0.0.1 benchmarks/moe_layer.py ...

Both arms receive the same tokens, routing, gates and expert weights (converted between the two weight layouts) and
compute  out[t] = sum_k gate[t,k] * Expert_{eid[t,k]}(x[t]).  Ours: ``Rdep.moe`` (nmoe_b200/parallel/rdep.py).
Reference: its stock ``nmoe.rdep.Rdep(...).moe_bf16`` / ``.moe_blockscaled`` (nmoe/rdep.py:34-145, nmoe/moe.py:52-617)
from the installation under baseline/_ref, the path its own nmoe/bench_moe_e2e.py:58-104 times.  Each iteration is
timed on the device with CUDA events after an L2 flush and a barrier; the figure is the mean over iterations, max
over ranks.  One JSON line per configuration with both times, their ratio and the largest output difference.

The reference's block-scaled profiles need its CuTe-DSL grouped GEMM, whose file only travels to one-GPU boxes.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

SHAPES = {"moonlight": dict(hidden=2048, inter=1408, experts=64, topk=6),
          "dsv3": dict(hidden=7168, inter=2048, experts=256, topk=8)}


def zipf_routing(T, E, K, s, gen, dev):
  p = (torch.arange(1, E + 1, dtype=torch.float64, device=dev) ** -s)
  p = (p / p.sum()).float()
  return torch.multinomial(p.expand(T, E), K, replacement=False, generator=gen).int()


def main():
  ap = argparse.ArgumentParser()
  ap.add_argument("--shape", default="moonlight", choices=sorted(SHAPES))
  ap.add_argument("--tokens", default="16384", help="tokens per rank, comma separated")
  ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp8", "nvfp4"])
  ap.add_argument("--routing", default="uniform", choices=["uniform", "zipf"])
  ap.add_argument("--impl", default="both", choices=["both", "ours", "reference"])
  ap.add_argument("--backward", action="store_true", help="time forward + backward instead of forward")
  ap.add_argument("--iters", type=int, default=10)
  ap.add_argument("--warmup", type=int, default=3)
  a = ap.parse_args()

  world = int(os.environ.get("WORLD_SIZE", "1"))
  rank = int(os.environ.get("RANK", "0"))
  local = int(os.environ.get("LOCAL_RANK", "0"))
  torch.cuda.set_device(local)
  dev = torch.device("cuda", local)
  if world > 1:
    dist.init_process_group("nccl", device_id=dev)
  sh = SHAPES[a.shape]
  H, F, E, K = sh["hidden"], sh["inter"], sh["experts"], sh["topk"]
  n_local = E // world
  sizes = [int(t) for t in a.tokens.split(",")]
  gen = torch.Generator(device=dev)
  gen.manual_seed(1234 + rank)
  W13 = (torch.randn(n_local, 2 * F, H, device=dev, generator=gen) * 0.02).bfloat16()
  W2 = (torch.randn(n_local, H, F, device=dev, generator=gen) * 0.02).bfloat16()
  flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

  def barrier():
    if world > 1:
      dist.barrier()
    torch.cuda.synchronize()

  def timed(fn):
    for _ in range(a.warmup):
      fn()
    barrier()
    tot = 0.0
    for _ in range(a.iters):
      flush.zero_()
      barrier()
      e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
      e0.record()
      fn()
      e1.record()
      torch.cuda.synchronize()
      tot += e0.elapsed_time(e1)
    t = torch.tensor([tot / a.iters], device=dev, dtype=torch.float64)
    if world > 1:
      dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())

  ours = ref = None
  ref_why = None
  if a.impl in ("both", "ours"):
    from nmoe_b200.ops import tc_gemm as G
    from nmoe_b200.ops.quant import ExpertWeightCache
    from nmoe_b200.parallel.rdep import Rdep
    ours = Rdep(H, E, K, max(sizes), device=dev, profile=a.dtype)
    W13o = W13.clone().requires_grad_(a.backward)
    W2o = W2.clone().requires_grad_(a.backward)
    wq = ExpertWeightCache(a.dtype).get(W13o, W2o) if a.dtype != "bf16" else None
  if a.impl in ("both", "reference"):
    try:
      from baseline import ref_arm, ref_env
      from nmoe_b200.parallel.rdep import to_reference_layout
      ref = ref_arm.RefMoELayer(H, F, E, K, max(sizes), profile=a.dtype)
      W1r, W3r, W2r = to_reference_layout(W13, W2)
      with torch.no_grad():
        ref.W1.copy_(W1r); ref.W3.copy_(W3r); ref.W2.copy_(W2r)
      if ref.cache is not None:
        from nmoe.blockscaled.grouped import quantize_weights
        ref.cache = quantize_weights(ref.W1, ref.W3, ref.W2, profile=a.dtype)
      del W1r, W3r, W2r
    except Exception as e:  # noqa: BLE001
      ref, ref_why = None, f"{type(e).__name__}: {' '.join(str(e).split())[:300]}"

  try:
    for T in sizes:
      x = (torch.randn(T, H, device=dev, generator=gen) * 0.5).bfloat16()
      if a.routing == "uniform":
        eid = torch.rand(T, E, device=dev, generator=gen).topk(K, dim=-1).indices.int()
      else:
        eid = zipf_routing(T, E, K, 1.2, gen, dev)
      gates = torch.rand(T, K, device=dev, generator=gen)
      gates = (gates / gates.sum(-1, keepdim=True)).contiguous()
      gout = torch.randn(T, H, device=dev, generator=gen).bfloat16()
      rec = {"bench": "moe_layer", "shape": a.shape, "n_gpus": world, "dtype": a.dtype, "routing": a.routing,
             "tokens_per_rank": T, "hidden": H, "inter": F, "experts": E, "topk": K, "backward": a.backward,
             "iters": a.iters, "l2": "256 MiB buffer written between iterations"}
      y_o = y_r = None
      if ours is not None:
        xo = x.clone().requires_grad_(a.backward)

        def f_ours():
          o = ours.moe(xo, gates, eid, W13o, W2o, False, wq)
          if a.backward:
            xo.grad = None; W13o.grad = None; W2o.grad = None
            o.backward(gout)
          return o
        rec["ours_ms"] = timed(f_ours)
        G.check_status()
        with torch.no_grad():
          y_o = ours.moe(x, gates, eid, W13o, W2o, False, wq).float()
      if ref is not None:
        xr = x.clone().requires_grad_(a.backward)
        gb = gates.bfloat16()
        el = eid.long()

        def f_ref():
          o = ref.forward(xr, el, gb)
          if a.backward:
            xr.grad = None; ref.W1.grad = None; ref.W3.grad = None; ref.W2.grad = None
            o.backward(gout)
          return o
        try:
          rec["reference_ms"] = timed(f_ref)
          with torch.no_grad():
            y_r = ref.forward(x, el, gb).float()
        except Exception as e:  # noqa: BLE001
          ref_why = f"{type(e).__name__}: {' '.join(str(e).split())[:300]}"
      if ref_why:
        rec["reference_unavailable"] = ref_why
      if "ours_ms" in rec and "reference_ms" in rec:
        rec["speedup_vs_reference"] = rec["reference_ms"] / rec["ours_ms"]
      if y_o is not None and y_r is not None:
        rec["max_abs_diff_vs_reference"] = (y_o - y_r).abs().max().item()
        rec["output_abs_max"] = y_r.abs().max().item()
      fl = 2.0 * T * K * 3 * H * F * (3 if a.backward else 1)
      if "ours_ms" in rec:
        rec["ours_tflops_per_gpu"] = fl / rec["ours_ms"] / 1e9
      if rank == 0:
        if ref is not None:
          rec["substitutions"] = ref_env.substitutions()
        print(json.dumps(rec), flush=True)
  finally:
    if ours is not None:
      ours.close()
    if world > 1:
      dist.destroy_process_group()


if __name__ == "__main__":
  main()
