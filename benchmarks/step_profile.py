"""Device time of one Moonlight-16B-A3B training step by kernel (one GPU, torch profiler, CUDA activity only).

  python benchmarks/step_profile.py [--dtype fp8|bf16] [--top 40] [--gaps 20] [--activation-checkpoint none|attention] [--recompute-h13]

Three warm-up steps, then one profiled step; prints the summed device time, and per kernel name the
total milliseconds and the launch count.  Times under the profiler are a few percent higher than
in a free run; use the shares, and ``bench.py`` for the step time itself.  ``--gaps N`` also lists where the
device sat idle: the N largest sums of idle time, keyed by the kernel that ran before and the one that ran after.
"""
from __future__ import annotations

import argparse
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch  # noqa: E402
from torch.profiler import ProfilerActivity, profile  # noqa: E402


def main():
  ap = argparse.ArgumentParser()
  ap.add_argument("--top", type=int, default=40)
  ap.add_argument("--gaps", type=int, default=0)
  ap.add_argument("--activation-checkpoint", default="none")
  ap.add_argument("--recompute-h13", action="store_true")
  ap.add_argument("--dtype", default="fp8", choices=["bf16", "fp8", "nvfp4"], help="expert GEMM profile")
  a = ap.parse_args()
  import bench
  from nmoe_b200 import runtime
  from nmoe_b200.train import Trainer
  rank, world, device = runtime.init(42)
  cfg = bench.moonlight_cfg(1, 4, 4096, a.dtype, None, a.activation_checkpoint, not a.recompute_h13)
  tr = Trainer(cfg, rank=rank, world=world, device=device)
  gen = torch.Generator().manual_seed(1234)

  def batch():
    h = torch.randint(0, cfg.vocab_size - 1, (4, 4097), generator=gen)
    return h[:, :-1].contiguous().to(device), h[:, 1:].contiguous().to(device)

  for _ in range(3):
    tr.step(*batch())
  torch.cuda.synchronize()
  x, y = batch()
  with profile(activities=[ProfilerActivity.CUDA]) as prof:
    tr.step(x, y)
    torch.cuda.synchronize()
  ev = prof.key_averages()
  total = sum(e.device_time_total for e in ev)
  print(f"total device ms {total / 1e3:.1f}")
  for e in sorted(ev, key=lambda e: -e.device_time_total)[:a.top]:
    print(f"{e.device_time_total / 1e3:8.2f} ms {e.count:6d}  {e.key[:120]}")
  if a.gaps > 0:
    from torch.autograd import DeviceType
    ks = sorted((e for e in prof.events() if e.device_type == DeviceType.CUDA and e.time_range is not None),
                key=lambda e: e.time_range.start)
    idle, by_pair, busy_end = 0.0, {}, None
    prev = None
    for e in ks:
      st, en = e.time_range.start, e.time_range.end
      if busy_end is not None and st > busy_end:
        g = st - busy_end
        idle += g
        key = (prev.name[:60], e.name[:60])
        c = by_pair.setdefault(key, [0.0, 0, 0.0])
        c[0] += g; c[1] += 1; c[2] = max(c[2], g)
      if busy_end is None or en > busy_end:
        busy_end, prev = en, e
    print(f"idle device ms {idle / 1e3:.2f} over {len(ks)} kernels")
    for (pa, pb), (g, n, mx) in sorted(by_pair.items(), key=lambda kv: -kv[1][0])[:a.gaps]:
      print(f"{g / 1e3:8.3f} ms {n:5d} gaps (max {mx:7.1f} us)  {pa}  ->  {pb}")
  if tr.model.rdep is not None:
    tr.model.rdep.close()


if __name__ == "__main__":
  main()
