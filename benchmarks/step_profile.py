"""Device time of one Moonlight-16B-A3B training step by kernel (one GPU, torch profiler, CUDA activity only).

  python benchmarks/step_profile.py [--top 40] [--activation-checkpoint none|attention] [--recompute-h13]

Three warm-up steps, then one profiled step; prints the summed device time, and per kernel name the
total milliseconds and the launch count.  Times under the profiler are a few percent higher than
in a free run; use the shares, and ``bench.py`` for the step time itself.
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
  ap.add_argument("--activation-checkpoint", default="none")
  ap.add_argument("--recompute-h13", action="store_true")
  a = ap.parse_args()
  import bench
  from nmoe_b200 import runtime
  from nmoe_b200.train import Trainer
  rank, world, device = runtime.init(42)
  cfg = bench.moonlight_cfg(1, 4, 4096, "bf16", None, a.activation_checkpoint, not a.recompute_h13)
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
  if tr.model.rdep is not None:
    tr.model.rdep.close()


if __name__ == "__main__":
  main()
