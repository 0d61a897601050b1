"""Headline benchmark: training throughput (tokens/s, MFU) of Moonlight-16B-A3B.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
  python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
      --master-port P bench.py --gpus N --steps K --warmup W

Weak scaling: every GPU trains a micro-batch of 4 x 4096 synthetic tokens (uniform random ids,
random-init weights), experts are spread over the N GPUs with RDEP, everything else is ZeRO-2.
Rank 0 prints ONE JSON line.  `value` is the whole-job tokens/s timed on the device (CUDA events,
max over ranks) with the inputs already resident; `e2e` repeats the measurement through
`Trainer.step` with a pinned-host -> device copy of the inputs and a device -> host read of the
loss every step.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

PLANNING_HINT_TOK_S_PER_GPU = 30_000.0   # configs/flow_profiles.toml duration hints of the reference (not a measurement)


def moonlight_cfg(n_gpus: int, micro_batch: int, seq_len: int, dtype: str, layers: int | None = None,
                  activation_checkpoint: str = "none", save_h13: bool = True, overlap_shared: str = "auto"):
  from nmoe_b200.config import Config
  return Config(
    preset="moonlight", vocab_size=163840, eos_token_id=163839, dim=2048, inter_dim=11264, moe_inter_dim=1408,
    n_layers=layers or 27, n_dense_layers=1, n_heads=16, n_routed_experts=64, n_shared_experts=2,
    n_activated_experts=6, route_scale=2.446, q_lora_rank=1536, kv_lora_rank=512, qk_nope_head_dim=128,
    qk_rope_head_dim=64, v_head_dim=128, attn="mla", attn_global_every=1, dtype=dtype, lr_dense=3e-4, lr_router=3e-4,
    lr_expert=3e-4, batch_size=micro_batch * n_gpus, seq_len=seq_len, warmup_steps=500, seed=42,
    activation_checkpoint=activation_checkpoint, moe_save_h13=save_h13, moe_overlap_shared=overlap_shared)


class ClockSampler:
  """nvidia-smi clock / throttle-reason sampler running for the duration of the timed region (read-only)."""
  Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
       "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
       "clocks_event_reasons.sw_power_cap")

  def __init__(self, gpu_index: int):
    self.f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
    self.p = None
    self.idx = gpu_index

  def start(self):
    try:
      self.p = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200",
                                 "-i", str(self.idx)], stdout=self.f, stderr=subprocess.DEVNULL)
    except OSError:
      self.p = None

  def stop(self) -> dict:
    if self.p is None:
      return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
    self.p.terminate()
    try:
      self.p.wait(timeout=5)
    except subprocess.TimeoutExpired:
      self.p.kill()
    self.f.flush()
    self.f.seek(0)
    sm, mx, reasons = [], [], set()
    names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
    for line in self.f.read().splitlines():
      parts = [x.strip() for x in line.split(",")]
      if len(parts) < 9:
        continue
      try:
        sm.append(float(parts[1]))
        mx.append(float(parts[2]))
      except ValueError:
        continue
      for n, v in zip(names, parts[5:9]):
        if v.lower().startswith("active"):
          reasons.add(n)
    os.unlink(self.f.name)
    if not sm:
      return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
    busy = [s for s in sm if s > 0]
    return {"sm_mhz": statistics.median(busy), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def flops_per_token(cfg) -> float:
  """Training FLOPs per token as in the reference's MFU accounting (nmoe/metrics.py:69-124):
  6 * active parameters (without the embedding table) + 6 * L * heads * (nope + rope + v) * seq."""
  H, L = cfg.dim, cfg.n_layers
  attn = (H * cfg.q_lora_rank + cfg.q_lora_rank * cfg.n_heads * cfg.qk_head_dim + H * (cfg.kv_lora_rank + cfg.qk_rope_head_dim)
          + cfg.kv_lora_rank * cfg.n_heads * (cfg.qk_nope_head_dim + cfg.v_head_dim) + cfg.n_heads * cfg.v_head_dim * H)
  dense_mlp = 3 * H * cfg.inter_dim
  l_moe = L - cfg.n_dense_layers
  moe_active = H * cfg.n_routed_experts + cfg.n_activated_experts * 3 * H * cfg.moe_inter_dim \
      + cfg.n_shared_experts * 3 * H * cfg.moe_inter_dim
  active = L * attn + cfg.n_dense_layers * dense_mlp + l_moe * moe_active + cfg.vocab_size * H
  return 6.0 * active + 6.0 * L * cfg.n_heads * (cfg.qk_nope_head_dim + cfg.qk_rope_head_dim + cfg.v_head_dim) * cfg.seq_len


def run_reference(args) -> None:
  """The unmodified reference through its own entry point.  It hard-requires its compiled
  `nmoe.csrc.rdep` extension plus FlashAttention-4 (`flash_attn.cute`) and FlashMLA for MLA
  (nmoe/attention/mla.py:66-72); when any of these cannot be imported the arm is unavailable."""
  why = None
  sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))
  try:
    import nmoe  # noqa: F401
  except Exception as e:
    why = f"reference package not installed under baseline/_ref: {type(e).__name__}: {e}"
  if why is None:
    for mod, what in (("nmoe.csrc.rdep", "compiled RDEP extension (its Makefile aborts without FlashMLA sources)"),
                      ("flash_attn.cute.interface", "FlashAttention-4 CuTe forward used by its MLA"),
                      ("nmoe.csrc.flashmla_sm100", "FlashMLA sm100 backward extension used by its MLA")):
      try:
        __import__(mod)
      except Exception as e:
        why = f"{mod} not importable ({what}): {type(e).__name__}"
        break
  if why is None:
    try:
      from nmoe.train import train as ref_train  # noqa: F401
      why = "reference imports succeeded but its trainer needs pre-tokenized shards under data_path; no synthetic-data entry point"
    except Exception as e:
      why = f"nmoe.train not importable: {type(e).__name__}: {e}"
  if int(os.environ.get("RANK", "0")) == 0:
    print(json.dumps({"impl": "reference", "unavailable": why}))


def main() -> None:
  ap = argparse.ArgumentParser()
  ap.add_argument("--gpus", type=int, default=1)
  ap.add_argument("--steps", type=int, default=5)
  ap.add_argument("--warmup", type=int, default=3)
  ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
  ap.add_argument("--micro-batch", type=int, default=4)
  ap.add_argument("--seq-len", type=int, default=4096)
  ap.add_argument("--layers", type=int, default=None, help="debug only: fewer layers (result is marked invalid)")
  ap.add_argument("--dtype", default="bf16")
  ap.add_argument("--no-e2e", action="store_true")
  ap.add_argument("--overlap-shared", default="auto", choices=["auto", "0", "1"], help="shared-expert MLP on a second stream")
  ap.add_argument("--recompute-h13", action="store_true", help="recompute the experts' up/gate output in backward (saves ~16 GB on one GPU)")
  ap.add_argument("--activation-checkpoint", default="none", choices=["none", "attention", "full"],
                  help="activation recompute policy; 'none' keeps the ~4 GB of attention activations instead of recomputing them")
  args = ap.parse_args()
  if args.impl == "reference":
    run_reference(args)
    return

  import torch
  import torch.distributed as dist
  from nmoe_b200 import runtime
  from nmoe_b200.ops import _lib, tc_gemm
  from nmoe_b200.train import Trainer

  world_env = int(os.environ.get("WORLD_SIZE", "1"))
  if world_env != args.gpus:
    if args.gpus > 1 and world_env == 1:
      raise SystemExit("--gpus N>1 must be launched with torch.distributed.run (one rank per GPU)")
  rank, world, device = runtime.init(42)
  cfg = moonlight_cfg(world, args.micro_batch, args.seq_len, args.dtype, args.layers, args.activation_checkpoint,
                      not args.recompute_h13, args.overlap_shared)
  trainer = Trainer(cfg, rank=rank, world=world, device=device)
  mb, S = args.micro_batch, args.seq_len
  gen = torch.Generator().manual_seed(1234 + rank)
  n_batches = args.warmup + args.steps
  host = [torch.randint(0, cfg.vocab_size - 1, (mb, S + 1), generator=gen) for _ in range(n_batches)]
  host_x = [h[:, :-1].contiguous().pin_memory() for h in host]
  host_y = [h[:, 1:].contiguous().pin_memory() for h in host]

  def barrier():
    if world > 1:
      dist.barrier()
    torch.cuda.synchronize()

  def max_over_ranks(ms: float) -> float:
    if world == 1:
      return ms
    t = torch.tensor([ms], device=device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())

  # ---- device-timed kernel path: inputs resident on the device, no host read inside the region
  dev_x = [x.to(device) for x in host_x]
  dev_y = [y.to(device) for y in host_y]
  for i in range(args.warmup):
    trainer.step(dev_x[i], dev_y[i])
  barrier()
  tc_gemm.check_status()
  sampler = ClockSampler(device.index or 0)
  if rank == 0:
    sampler.start()
  _lib.reset_launch_count()
  ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
  barrier()
  ev0.record()
  for i in range(args.steps):
    loss = trainer.step(dev_x[args.warmup + i], dev_y[args.warmup + i])
  ev1.record()
  barrier()
  launches = _lib.launch_count()
  ms = max_over_ranks(ev0.elapsed_time(ev1))
  clocks = sampler.stop() if rank == 0 else None
  final_loss = float(loss.item())
  tc_gemm.check_status()
  tokens = world * mb * S * args.steps
  tok_s = tokens / (ms / 1e3)
  peak_alloc = torch.cuda.max_memory_allocated() / 2 ** 30

  # ---- end to end through Trainer.step: pinned host inputs copied every step, loss read back every step
  e2e = None
  if not args.no_e2e:
    barrier()
    t0 = time.perf_counter()
    ev0.record()
    for i in range(args.steps):
      l = trainer.step(host_x[args.warmup + i], host_y[args.warmup + i])
      _ = l.item()
    ev1.record()
    barrier()
    wall_ms = (time.perf_counter() - t0) * 1e3
    e_ms = max_over_ranks(max(ev0.elapsed_time(ev1), wall_ms))
    e2e = {"value": tokens / (e_ms / 1e3), "unit": "tokens/s", "h2d_bytes_per_step": int(2 * mb * S * 8 * world),
           "d2h_bytes_per_step": int(4 * world), "ms_per_step": e_ms / args.steps}

  if rank == 0:
    peaks = {}
    try:
      peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except OSError:
      pass
    fpt = flops_per_token(cfg)
    tflops_per_gpu = tok_s / world * fpt / 1e12
    out = {
      "metric": "training throughput, Moonlight-16B-A3B (tokens/s whole job; MFU alongside)",
      "value": tok_s, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
      "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
      "dtype": args.dtype, "data": "synthetic uniform-random token ids, random-init weights",
      "config": {"model": "moonlight-16b-a3b" if args.layers is None else f"INVALID-debug-{args.layers}-layers",
                 "global_batch": world * mb, "seq_len": S,
                 "parallelism": (f"rdep-ep{world}+zero2-dp{world}" if world > 1 else "single-gpu"),
                 "vocab": cfg.vocab_size, "layers": cfg.n_layers, "experts": "64 top-6 + 2 shared",
                 "activation_checkpoint": args.activation_checkpoint, "moe_save_h13": not args.recompute_h13,
                 "l2": "per-step working set (32 GB of weights) is far larger than the 126 MB L2"},
      "tflops_per_gpu": tflops_per_gpu,
      "mfu_vs_nominal_2250": tflops_per_gpu / 2250.0,
      "mfu_vs_measured_sustained": (tflops_per_gpu / peaks["bf16_tflops_sustained"]) if peaks else None,
      "vs_reference_planning_hint_30k_tok_s_per_gpu": tok_s / world / PLANNING_HINT_TOK_S_PER_GPU,
      "final_loss": final_loss, "peak_mem_gib": peak_alloc, "clocks": clocks, "e2e": e2e,
      "gpu_launches": launches, "zero2_impl": trainer.opt.dense.impl,
    }
    print(json.dumps(out))
  if trainer.model.rdep is not None:
    trainer.model.rdep.close()
  runtime.finalize()


if __name__ == "__main__":
  main()
