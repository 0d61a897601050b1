"""RDEP micro-benchmark: dispatch -> grouped GEMMs -> fused return on an expert shape, per phase.

  torchrun --nnodes 1 --nproc-per-node N --master-addr 127.0.0.1 benchmarks/rdep.py \
      [--hidden 7168 --inter 2048 --experts 256 --topk 8] [--tokens 512,4096,32768] [--dtype bf16|fp8|nvfp4]
      [--routing uniform|zipf] [--iters 10 --warmup 3]

(also runs with plain ``python`` on one GPU).  Every phase is timed on the device with CUDA events
after a barrier; the reported time is the max over ranks.  One JSON line per token count:

  dispatch_us   count + plan (count exchange over peer stores) + placement stores into the owners'
                buffers (quantising for fp8 / nvfp4) + wait for every source's data flag
  gemm13_us     grouped up/gate projection + SwiGLU (fused quantise for fp8 / nvfp4)
  gemm2_ret_us  grouped down projection whose epilogue streams each (expert, source) run of rows into the
                source's return buffer, + flag exchange + the gate-weighted K-way sum at the source
  nvlink_gbs    bytes this rank stored to OTHER ranks during dispatch and return / their time
                (fraction of the 900 GB/s per-direction link also given)

The counterpart in the reference is tests/bench_rdep_kernels.py (dispatch / gather latency) and
nmoe/bench_moe_e2e.py (p50 forward).  ``--routing zipf`` draws experts from a Zipf(s=1.2) law, the
skewed case of the reference's worst-case test.
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


def zipf_routing(T: int, E: int, K: int, s: float, gen: torch.Generator, dev) -> torch.Tensor:
  """K distinct experts per token, drawn without replacement from p(e) ~ (e+1)^-s."""
  p = (torch.arange(1, E + 1, dtype=torch.float64, device=dev) ** -s)
  p = (p / p.sum()).float()
  return torch.multinomial(p.expand(T, E), K, replacement=False, generator=gen).int()


def main():
  ap = argparse.ArgumentParser()
  ap.add_argument("--hidden", type=int, default=7168)
  ap.add_argument("--inter", type=int, default=2048)
  ap.add_argument("--experts", type=int, default=256)
  ap.add_argument("--topk", type=int, default=8)
  ap.add_argument("--tokens", default="512,4096,16384")
  ap.add_argument("--dtype", default="bf16")
  ap.add_argument("--routing", default="uniform", choices=["uniform", "zipf"])
  ap.add_argument("--iters", type=int, default=10)
  ap.add_argument("--warmup", type=int, default=3)
  ap.add_argument("--capacity-factor", type=float, default=2.0)
  ap.add_argument("--detail", action="store_true",
                  help="unfused return only: also time the down GEMM, the push kernel, the flag wait and the K-way sum, "
                       "with a barrier before the push so that rank skew does not count as push time")
  a = ap.parse_args()

  world = int(os.environ.get("WORLD_SIZE", "1"))
  rank = int(os.environ.get("RANK", "0"))
  local = int(os.environ.get("LOCAL_RANK", "0"))
  torch.cuda.set_device(local)
  dev = torch.device("cuda", local)
  if world > 1:
    dist.init_process_group("nccl", device_id=dev)

  from nmoe_b200.ops import elementwise as EW
  from nmoe_b200.ops import quant as Q
  from nmoe_b200.ops import tc_gemm as G
  from nmoe_b200.parallel.rdep import Rdep

  H, F, E, K = a.hidden, a.inter, a.experts, a.topk
  n_local = E // world
  sizes = [int(t) for t in a.tokens.split(",")]
  gen = torch.Generator(device=dev)
  gen.manual_seed(1234 + rank)
  W13 = (torch.randn(n_local, 2 * F, H, device=dev) * 0.02).bfloat16()
  W2 = (torch.randn(n_local, H, F, device=dev) * 0.02).bfloat16()
  quantised = a.dtype != "bf16"
  wq = Q.ExpertWeightCache(a.dtype).get(W13, W2) if quantised else None
  # zipf needs room for the hot experts' owner to receive most rows
  cf = a.capacity_factor if a.routing == "uniform" else float(world)
  rd = Rdep(H, E, K, max(sizes), capacity_factor=cf, device=dev, profile=a.dtype)
  flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

  def barrier():
    if world > 1:
      dist.barrier()
    torch.cuda.synchronize()

  try:
    for T in sizes:
      x = torch.randn(T, H, device=dev, generator=gen).bfloat16()
      if a.routing == "uniform":
        eid = torch.rand(T, E, device=dev, generator=gen).topk(K, dim=-1).indices.int()
      else:
        eid = zipf_routing(T, E, K, 1.2, gen, dev)
      gates = torch.rand(T, K, device=dev, generator=gen)
      gates = (gates / gates.sum(-1, keepdim=True)).contiguous()
      out = torch.empty_like(x)
      remote_pairs = int(((eid // n_local) != rank).sum().item())
      ev = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(a.iters)]
      dv = [[torch.cuda.Event(enable_timing=True) for _ in range(5)] for _ in range(a.iters)]
      detail = a.detail and not rd.fused_return

      def one(marks, dmarks=None):
        if marks:
          marks[0].record()
        plan = rd.plan(eid)
        if quantised:
          rd.place_mx(x, plan, gates.view(-1))
        else:
          rd.place(x, plan, gates.view(-1), "x", with_meta=True)
        rd.wait_data()
        if marks:
          marks[1].record()
        if quantised:
          gg = Q.grouped_gemm_mxfp4 if rd.fp4 else Q.grouped_gemm_mxfp8
          aq, asf = Q.grouped_gemm_swiglu_quant(rd.xq, rd.sfa, wq[0], wq[1], plan.tile_expert, plan.n_m_tiles, fp4=rd.fp4)
        else:
          h13 = G.grouped_gemm(rd.xbuf, W13, plan.tile_expert, plan.n_m_tiles, align256=rd.align == 256)
          act = EW.swiglu_rows(h13, plan.n_m_tiles)
        if marks:
          marks[2].record()
        if not rd.fused_return:      # NMOE_RDEP_FUSED_RETURN=0: GEMM into a local buffer, then a separate push kernel
          if dmarks:
            dmarks[0].record()
          y = (gg(aq, asf, wq[2], wq[3], plan.tile_expert, plan.n_m_tiles) if quantised
               else G.grouped_gemm(act, W2, plan.tile_expert, plan.n_m_tiles, align256=rd.align == 256))
          if dmarks:
            dmarks[1].record()
            barrier()                      # every rank starts its push together
            dmarks[2].record()
          rd.push_and_reduce(y, plan, gates.view(-1), None, out, marks=dmarks[3:5] if dmarks else None)
        else:
          if quantised:
            gg(aq, asf, wq[2], wq[3], plan.tile_expert, plan.n_m_tiles, push=rd.push_args(plan))
          else:
            G.grouped_gemm(act, W2, plan.tile_expert, plan.n_m_tiles, push=rd.push_args(plan), align256=rd.align == 256)
          rd.finish_return(plan, out, gates.view(-1))
        if marks:
          marks[3].record()
        return plan

      for _ in range(a.warmup):
        one(None)
      barrier()
      G.check_status()
      for it in range(a.iters):
        flush.zero_()
        barrier()
        plan = one(ev[it], dv[it] if detail else None)
      barrier()
      G.check_status()
      rows_here = int(plan.offs_pad[-1].item())
      ph = torch.tensor([[e[i].elapsed_time(e[i + 1]) for i in range(3)] for e in ev], device=dev).mean(0) * 1e3
      if world > 1:
        dist.all_reduce(ph, op=dist.ReduceOp.MAX)
      d_us, g_us, r_us = ph.tolist()
      row_in = {"bf16": 2 * H, "fp8": H + H // 32}.get(a.dtype, H // 2 + H // 32) + 16
      sent = remote_pairs * (row_in + 2 * H + 4)          # dispatch out + (symmetric on average) return in
      comm_s = (d_us + r_us) * 1e-6
      flops = 2.0 * T * K * 3 * H * F
      # roofline of the fused down-projection + return: the slower of its FLOPs at the measured sustained GEMM
      # rate and its bytes over NVLink at the measured peer-copy rate (770 GB/s per direction)
      peak = {"bf16": 1424e12, "fp8": 2848e12}.get(a.dtype, 5696e12)
      try:
        pk = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        peak = pk["bf16_tflops_sustained"] * 1e12 * {"bf16": 1, "fp8": 2}.get(a.dtype, 4)
      except (OSError, KeyError):
        pass
      ret_floor_us = max(2.0 * rows_here * H * F / peak, remote_pairs * 2 * H / 770e9) * 1e6
      extra = {}
      if detail:
        dt = torch.tensor([[d[0].elapsed_time(d[1]), d[2].elapsed_time(d[3]), d[3].elapsed_time(d[4]),
                            d[4].elapsed_time(e[3])] for d, e in zip(dv, ev)], device=dev).mean(0) * 1e3
        if world > 1:
          dist.all_reduce(dt, op=dist.ReduceOp.MAX)
        g2, pu, wa, re = dt.tolist()
        extra = {"detail_us": {"gemm2": round(g2, 1), "push": round(pu, 1), "flag_wait": round(wa, 1),
                               "reduce": round(re, 1)},
                 "push_gbs_rank0": round(remote_pairs * 2 * H / (pu * 1e-6) / 1e9, 1) if world > 1 else 0.0,
                 "push_impl": "bulk" if rd.push_impl else "st.v4"}
      if rank == 0:
        print(json.dumps({
          "bench": "rdep", **extra, "n_gpus": world, "dtype": a.dtype, "routing": a.routing, "tokens_per_rank": T,
          "hidden": H, "inter": F, "experts": E, "topk": K, "padded_rows_rank0": rows_here,
          "dispatch_us": round(d_us, 1), "gemm13_us": round(g_us, 1), "gemm2_ret_us": round(r_us, 1),
          "total_us": round(d_us + g_us + r_us, 1),
          "gemm2_ret_roofline_us": round(ret_floor_us, 1), "gemm2_ret_frac_of_roofline": round(ret_floor_us / max(r_us, 1e-9), 3),
          "tflops_per_gpu": round(flops / ((d_us + g_us + r_us) * 1e-6) / 1e12, 1),
          "remote_pairs_rank0": remote_pairs,
          "nvlink_gbs_rank0": round(sent / comm_s / 1e9, 1) if world > 1 else 0.0,
          "frac_of_900": round(sent / comm_s / 900e9, 3) if world > 1 else 0.0,
        }), flush=True)
  finally:
    rd.close()
    if world > 1:
      dist.destroy_process_group()


if __name__ == "__main__":
  main()
