"""Kernel micro-benchmarks (device-timed with CUDA events, L2 flushed between iterations).

  python benchmarks/kernels.py gemm  --m 16384 --n 2048 --k 2048 [--a-mn] [--b-mn] [--bn 256]
  python benchmarks/kernels.py mx    --m 16384 --n 2816 --k 2048
  python benchmarks/kernels.py attn  --b 4 --s 4096 --h 16 --dqk 192 --dv 128 [--window 128]
  python benchmarks/kernels.py moe   --tokens 16384 --hidden 2048 --inter 1408 --experts 64 --topk 6 [--dtype fp8]

Each prints one JSON line with the time, achieved TFLOP/s or GB/s and the fraction of the measured
peak (MEASURED_PEAKS.json next to the repository root, if present).  ``--iters 1 --warmup 1`` keeps a
run short enough for a profiler capture.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch  # noqa: E402


def peaks():
  try:
    return json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
  except OSError:
    return {"bf16_tflops": 1590.0, "hbm_gbs": 6650.0, "fallback": True}


def timed(fn, iters, warmup, flush):
  for _ in range(warmup):
    fn()
  torch.cuda.synchronize()
  total = 0.0
  for _ in range(iters):
    if flush is not None:
      flush.zero_()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    fn()
    e.record()
    torch.cuda.synchronize()
    total += s.elapsed_time(e)
  return total / iters


def main():
  ap = argparse.ArgumentParser()
  ap.add_argument("what", choices=["gemm", "mx", "attn", "moe", "indexer", "elementwise", "adamwq", "kda", "sparse", "nsa"])
  for k, d in (("m", 16384), ("n", 2048), ("k", 2048), ("bn", 0), ("b", 4), ("s", 4096), ("h", 16), ("dqk", 192), ("dv", 128),
               ("window", 0), ("tokens", 16384), ("hidden", 2048), ("inter", 1408), ("experts", 64), ("topk", 6),
               ("idx-heads", 4), ("idx-dim", 64), ("iters", 20), ("warmup", 3)):
    ap.add_argument(f"--{k}", type=int, default=d)
  ap.add_argument("--a-mn", action="store_true"); ap.add_argument("--b-mn", action="store_true")
  ap.add_argument("--dtype", default="bf16"); ap.add_argument("--no-flush", action="store_true")
  ap.add_argument("--backward", action="store_true")
  a = ap.parse_args()
  from nmoe_b200 import ops
  from nmoe_b200.ops import tc_gemm as G
  dev = torch.device("cuda")
  pk = peaks()
  flush = None if a.no_flush else torch.empty(256 << 20, dtype=torch.uint8, device=dev)   # > 126 MB L2
  out = {"what": a.what}
  if a.what == "gemm":
    A = torch.randn((a.k, a.m) if a.a_mn else (a.m, a.k), device=dev).bfloat16()
    B = torch.randn((a.k, a.n) if a.b_mn else (a.n, a.k), device=dev).bfloat16()
    C = torch.empty(a.m, a.n, device=dev, dtype=torch.bfloat16)
    ms = timed(lambda: G.gemm(A, B, a_mn=a.a_mn, b_mn=a.b_mn, out=C, bn=a.bn), a.iters, a.warmup, flush)
    tf = 2.0 * a.m * a.n * a.k / ms / 1e9
    out.update(shape=[a.m, a.n, a.k], a_mn=a.a_mn, b_mn=a.b_mn, ms=ms, tflops=tf, frac_of_measured_bf16_peak=tf / pk["bf16_tflops"])
  elif a.what == "mx":
    A = torch.randn(a.m, a.k, device=dev).bfloat16(); B = (torch.randn(a.n, a.k, device=dev) * 0.1).bfloat16()
    C = torch.empty(a.m, a.n, device=dev, dtype=torch.bfloat16)
    if a.dtype in ("nvfp4", "mxfp4", "fp4"):
      from nmoe_b200.ops.quant import gemm_mxfp4
      aq, asf = ops.quant_mxfp4(A); bq, bsf = ops.quant_mxfp4(B)
      ms = timed(lambda: gemm_mxfp4(aq, asf, bq, bsf, out=C, bn=a.bn), a.iters, a.warmup, flush)
      mult = 4
    else:
      aq, asf = ops.quant_mxfp8(A); bq, bsf = ops.quant_mxfp8(B)
      ms = timed(lambda: ops.gemm_mxfp8(aq, asf, bq, bsf, out=C, bn=a.bn), a.iters, a.warmup, flush)
      mult = 2
    tf = 2.0 * a.m * a.n * a.k / ms / 1e9
    out.update(shape=[a.m, a.n, a.k], dtype=a.dtype, ms=ms, tflops=tf)
    out[f"frac_of_{mult}x_measured_bf16_peak"] = tf / (mult * pk["bf16_tflops"])
  elif a.what == "attn":
    from nmoe_b200.ops.attention import attention_forward
    q = torch.randn(a.b, a.s, a.h, a.dqk, device=dev).bfloat16(); k = torch.randn_like(q)
    v = torch.randn(a.b, a.s, a.h, a.dv, device=dev).bfloat16()
    keys = a.s / 2 if a.window == 0 else min(a.window, a.s / 2)
    if a.backward:
      # backward kernels alone (delta pre-pass + dK/dV + dQ): 2 recomputed and 3 gradient products
      from nmoe_b200.ops.attention import attention_backward
      o, lse = attention_forward(q, k, v, a.dqk ** -0.5, a.window)
      do = torch.randn_like(o)
      ms = timed(lambda: attention_backward(q, k, v, o, do, lse, a.dqk ** -0.5, a.window), a.iters, a.warmup, flush)
      tf = 2.0 * a.b * a.h * a.s * keys * (3 * a.dqk + 2 * a.dv) / ms / 1e9
      out["backward"] = True
    else:
      ms = timed(lambda: attention_forward(q, k, v, a.dqk ** -0.5, a.window), a.iters, a.warmup, flush)
      tf = 2.0 * a.b * a.h * a.s * keys * (a.dqk + a.dv) / ms / 1e9
    out.update(shape=[a.b, a.s, a.h, a.dqk, a.dv], window=a.window, ms=ms, tflops=tf, frac_of_measured_bf16_peak=tf / pk["bf16_tflops"])
  elif a.what == "adamwq":
    # expert AdamW that also writes the block-scaled copy of the new weights (one pass: 7 bf16 streams + the copy)
    from nmoe_b200.ops.quant import expert_adamw_quant_, sf_bytes
    rows, K = a.experts * 2 * a.inter, a.hidden
    fp4 = a.dtype in ("nvfp4", "mxfp4", "fp4")
    p_ = torch.randn(rows, K, device=dev).bfloat16(); g_ = torch.randn_like(p_) * 0.01
    m_ = torch.zeros_like(p_); v_ = torch.zeros_like(p_)
    q_ = torch.empty(rows, K // 2 if fp4 else K, dtype=torch.uint8, device=dev)
    sf_ = torch.empty(sf_bytes(rows, K), dtype=torch.uint8, device=dev)
    ms = timed(lambda: expert_adamw_quant_(p_, g_, m_, v_, q_, sf_, fp4, lr=1e-3, beta1=0.9, beta2=0.99, eps=1e-8,
                                           weight_decay=0.1, step=3), a.iters, a.warmup, flush)
    nbytes = rows * K * (14.0 + (0.5 if fp4 else 1.0) + 1.0 / 32)
    out.update(rows=rows, K=K, dtype=a.dtype, ms=ms, gbs=nbytes / ms / 1e6, frac_of_measured_hbm=nbytes / ms / 1e6 / pk["hbm_gbs"])
  elif a.what == "kda":
    # gated delta rule, chunk form: batched WY transform (library products) + the chunk-recurrence scan kernel
    from nmoe_b200.ops.kda import kda_chunk_scan, scan
    B, T, H, Dk, Dv = a.b, a.s, a.h, a.dqk, a.dv
    q = torch.randn(B, T, H, Dk, device=dev).requires_grad_(a.backward); k = torch.randn(B, T, H, Dk, device=dev)
    v = torch.randn(B, T, H, Dv, device=dev); g = -torch.rand(B, T, H, Dk, device=dev) * 0.1; beta = torch.rand(B, T, H, device=dev)
    def run():
      o = kda_chunk_scan(q, k, v, g, beta)
      if a.backward:
        q.grad = None
        o.sum().backward()
    ms = timed(run, a.iters, a.warmup, flush)
    n = T // 64
    U = torch.randn(B * H, n, 64, Dv, device=dev); P = torch.randn(B * H, n, 64, Dk, device=dev) * 0.05
    K2 = torch.randn(B * H, n, 64, Dk, device=dev) * 0.05; dec = torch.rand(B * H, n, Dk, device=dev)
    ms_scan = timed(lambda: scan(U, P, K2, dec), a.iters, a.warmup, flush)
    fl = 2.0 * B * H * n * 2 * 64 * Dk * Dv
    out.update(shape=[B, T, H, Dk, Dv], backward=a.backward, ms=ms, scan_kernel_ms=ms_scan, scan_tflops=fl / ms_scan / 1e9)
  elif a.what == "sparse":
    # token-sparse attention: per-query top-k bit mask (radix select) + masked tcgen05 attention, against dense causal
    from nmoe_b200.ops.attention import SparseMask, attention_forward
    q = torch.randn(a.b, a.s, a.h, a.dqk, device=dev).bfloat16(); k = torch.randn_like(q)
    v = torch.randn(a.b, a.s, a.h, a.dv, device=dev).bfloat16()
    scores = torch.randn(a.b, a.s, a.s, device=dev)
    topk = max(1, a.s // 4)
    ms_mask = timed(lambda: SparseMask.from_topk_scores(scores, topk), a.iters, a.warmup, flush)
    mask = SparseMask.from_topk_scores(scores, topk)
    ms_sparse = timed(lambda: attention_forward(q, k, v, a.dqk ** -0.5, 0, mask=mask), a.iters, a.warmup, flush)
    ms_dense = timed(lambda: attention_forward(q, k, v, a.dqk ** -0.5, 0), a.iters, a.warmup, flush)
    ms_sort = timed(lambda: scores.topk(topk, dim=-1), max(2, a.iters // 4), 1, flush)
    out.update(shape=[a.b, a.s, a.h, a.dqk, a.dv], top_k=topk, mask_topk_ms=ms_mask, torch_topk_ms=ms_sort,
               masked_attention_ms=ms_sparse, dense_attention_ms=ms_dense)
  elif a.what == "nsa":
    # compressed branch of native sparse attention (group-mean queries over MLP-compressed keys, block scores fused):
    # the kernels against the PyTorch statement of the same maths, forward and forward + backward
    from nmoe_b200.ops import nsa as N
    B, T, KV, D, l, d, blk = a.b, a.s, a.h, a.dv, 32, 16, 64
    Tc = (T - l) // d + 1
    mk = lambda *sh: torch.randn(*sh, device=dev).bfloat16().requires_grad_(a.backward)
    q, kc, vc = mk(B, T, KV, D), mk(B, Tc, KV, D), mk(B, Tc, KV, D)
    def run(fn):
      def f():
        o, sc = fn(q, kc, vc, cmp_len=l, cmp_stride=d, slc_block=blk, scale=D ** -0.5)
        if a.backward:
          for x in (q, kc, vc):
            x.grad = None
          o.float().sum().backward()
      return f
    ms = timed(run(N.cmp_attention), a.iters, a.warmup, flush)
    ms_ref = timed(run(N.cmp_attention_reference), max(2, a.iters // 4), 1, flush)
    out.update(shape=[B, T, KV, D], compressed_keys=Tc, backward=a.backward, ms=ms, statement_ms=ms_ref, speedup=ms_ref / ms)
  elif a.what == "elementwise":
    # the memory-bound kernels of a step on the benchmark's shapes: algorithmic bytes / time against the measured copy rate
    from nmoe_b200.ops.optim import adamw_flat_
    T, H, F = a.tokens, a.hidden, a.inter
    rows = T * a.topk
    x = torch.randn(T, H, device=dev).bfloat16().requires_grad_(True)
    wn = torch.ones(H, device=dev).bfloat16().requires_grad_(True)
    gy = torch.randn(T, H, device=dev).bfloat16()
    h13 = torch.randn(rows, 2 * F, device=dev).bfloat16().requires_grad_(True)
    ga = torch.randn(rows, F, device=dev).bfloat16()
    res = {}
    def rec(name, ms, nbytes):
      res[name] = {"ms": ms, "gbs": nbytes / ms / 1e6, "frac_of_measured_hbm": nbytes / ms / 1e6 / pk["hbm_gbs"]}
    rec("rmsnorm_fwd", timed(lambda: ops.rmsnorm(x, wn, 1e-6), a.iters, a.warmup, flush), 2.0 * T * H * 2)
    y = ops.rmsnorm(x, wn, 1e-6)
    def nb():
      x.grad = None; wn.grad = None
      y.backward(gy, retain_graph=True)
    rec("rmsnorm_bwd", timed(nb, a.iters, a.warmup, flush), 3.0 * T * H * 2)
    rec("swiglu_fwd", timed(lambda: ops.swiglu(h13), a.iters, a.warmup, flush), 3.0 * rows * F * 2)
    act = ops.swiglu(h13)
    def sb():
      h13.grad = None
      act.backward(ga, retain_graph=True)
    rec("swiglu_bwd", timed(sb, a.iters, a.warmup, flush), 5.0 * rows * F * 2)
    n = 1 << 28
    pw = torch.randn(n, device=dev).bfloat16(); g = torch.randn(n, device=dev).bfloat16()
    m = torch.zeros(n, device=dev, dtype=torch.bfloat16); v = torch.zeros_like(m)
    rec("adamw_flat_256M", timed(lambda: adamw_flat_(pw, g, m, v, lr=1e-3, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, step=3),
                                 a.iters, a.warmup, flush), 7.0 * n * 2)
    out.update(tokens=T, hidden=H, inter=F, rows=rows, kernels=res)
  elif a.what == "indexer":
    # sparse-attention indexer scores: fused GEMM + relu + head sum against the eager statement
    from nmoe_b200.ops.indexer import indexer_scores, indexer_scores_ref
    q = torch.randn(a.b, a.s, a.idx_heads, a.idx_dim, device=dev).bfloat16()
    k = torch.randn(a.b, a.s, a.idx_dim, device=dev).bfloat16()
    w = torch.randn(a.b, a.s, a.idx_heads, device=dev).bfloat16()
    ms = timed(lambda: indexer_scores(q, k, w, True), a.iters, a.warmup, flush)
    ms_ref = timed(lambda: indexer_scores_ref(q, k, w, True), max(2, a.iters // 5), 1, flush)
    out_bytes = 4.0 * a.b * a.s * a.s
    out.update(shape=[a.b, a.s, a.idx_heads, a.idx_dim], ms=ms, eager_ms=ms_ref, speedup=ms_ref / ms,
               tflops=2.0 * a.b * a.s * (a.s / 2) * a.idx_heads * a.idx_dim / ms / 1e9,
               output_gbs=out_bytes / ms / 1e6, frac_of_measured_hbm=out_bytes / ms / 1e6 / pk["hbm_gbs"])
  else:
    from nmoe_b200.ops.quant import ExpertWeightCache
    from nmoe_b200.parallel.rdep import Rdep
    T, H, F, E, K = a.tokens, a.hidden, a.inter, a.experts, a.topk
    rd = Rdep(H, E, K, T, device=dev, profile=a.dtype)
    x = (torch.randn(T, H, device=dev) * 0.5).bfloat16().requires_grad_(a.backward)
    W13 = (torch.randn(E, 2 * F, H, device=dev) * 0.02).bfloat16().requires_grad_(a.backward)
    W2 = (torch.randn(E, H, F, device=dev) * 0.02).bfloat16().requires_grad_(a.backward)
    eid = torch.stack([torch.randperm(E, device=dev)[:K] for _ in range(min(T, 4096))]).int().repeat((T + 4095) // 4096, 1)[:T].contiguous()
    gates = torch.rand(T, K, device=dev)
    wq = ExpertWeightCache(a.dtype).get(W13, W2) if a.dtype != "bf16" else None
    g = torch.randn(T, H, device=dev).bfloat16()
    def step():
      o = rd.moe(x, gates, eid, W13, W2, False, wq)
      if a.backward:
        o.backward(g)
    ms = timed(step, a.iters, a.warmup, flush)
    # latency distribution (one event pair per call, L2 flushed in between), as the reference's MoE benchmark reports
    lat = sorted(timed(step, 1, 0, flush) for _ in range(max(a.iters, 20)))
    fl = 2.0 * T * K * 3 * H * F * (3 if a.backward else 1) + (2.0 * T * K * 2 * F * H if a.backward else 0)
    out.update(tokens=T, hidden=H, inter=F, experts=E, topk=K, dtype=a.dtype, backward=a.backward, ms=ms, tflops=fl / ms / 1e9,
               p50_ms=lat[len(lat) // 2], p99_ms=lat[min(len(lat) - 1, int(len(lat) * 0.99))])
    if a.dtype != "bf16":
      # accuracy of the block-scaled forward against the bf16 forward on the same inputs
      with torch.no_grad():
        y = rd.moe(x, gates, eid, W13, W2, False, wq).float()
      rd.close()
      rb = Rdep(H, E, K, T, device=dev, profile="bf16")
      with torch.no_grad():
        yb = rb.moe(x, gates, eid, W13, W2, False, None).float()
      rd = rb
      out.update(cos_vs_bf16=torch.nn.functional.cosine_similarity(y.flatten(), yb.flatten(), dim=0).item(),
                 max_abs_err=(y - yb).abs().max().item(), rel_err=((y - yb).norm() / yb.norm()).item())
    rd.close()
  G.check_status()
  print(json.dumps(out))


if __name__ == "__main__":
  main()
