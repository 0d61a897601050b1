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


MOONLIGHT_REF_FIELDS = dict(
  preset="moonlight", vocab_size=163840, eos_token_id=163839, dim=2048, inter_dim=11264, moe_inter_dim=1408, n_layers=27,
  n_dense_layers=1, n_heads=16, n_routed_experts=64, n_shared_experts=2, n_activated_experts=6, route_scale=2.446,
  q_lora_rank=1536, kv_lora_rank=512, qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128, attn="mla",
  attn_global_every=1, lr_dense=3e-4, lr_router=3e-4, lr_expert=3e-4, warmup_steps=500)


class _FailFlag:
  """Lets every rank of the reference arm leave when one of them fails: the failing rank writes its reason to a file
  keyed on the rendezvous port, a watcher thread in each other rank sees it within a second and exits the process, so
  no rank is left waiting in a collective.  Rank 0 prints the `unavailable` line."""

  def __init__(self, rank: int, deadline_s: float):
    import threading
    self.rank = rank
    self.path = os.path.join(tempfile.gettempdir(), f"nmoe_bench_ref_fail_{os.environ.get('MASTER_PORT', '0')}_{os.getppid()}")
    if rank == 0 and os.path.exists(self.path):
      os.unlink(self.path)
    self.deadline = time.time() + deadline_s
    self.done = False
    self.lock = threading.Lock()
    self.t = threading.Thread(target=self._watch, daemon=True)
    self.t.start()

  def _emit_and_exit(self, why: str):
    with self.lock:   # never released: the first caller prints and ends the process
      if self.rank == 0:
        print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)
      os._exit(0)

  def _watch(self):
    while not self.done:
      time.sleep(0.5)
      if os.path.exists(self.path):
        time.sleep(0.2)
        try:
          why = open(self.path).read().strip() or "another rank failed"
        except OSError:
          why = "another rank failed"
        self._emit_and_exit(why)
      if time.time() > self.deadline:
        self._emit_and_exit("reference arm exceeded its time limit (no step completed in time)")

  def fail(self, why: str):
    why = " ".join(str(why).split())[:400]
    try:
      with open(self.path, "x") as f:
        f.write(why)
    except OSError:
      pass
    self._emit_and_exit(why)

  def finish(self):
    self.done = True


def run_reference(args) -> None:
  """The unmodified reference (installed under baseline/_ref with its compiled RDEP extension) on the same model,
  batch and synthetic data, through its own Config / Transformer / loader / optimizer objects; see baseline/ref_arm.py.
  Its MLA needs FlashAttention-4 and FlashMLA, neither of which exists on this image; baseline/ref_env.py supplies
  cuDNN's fused attention under those two names and the JSON line says so in `substitutions`."""
  rank = int(os.environ.get("RANK", "0"))
  world_env = int(os.environ.get("WORLD_SIZE", "1"))
  flag = _FailFlag(rank, deadline_s=float(os.environ.get("NMOE_REF_ARM_DEADLINE_S", "1500")))
  try:
    from baseline import ref_arm, ref_env
    dtype = args.ref_dtype
    sampler = ClockSampler(int(os.environ.get("LOCAL_RANK", "0")))
    fields = dict(MOONLIGHT_REF_FIELDS)
    if args.layers:
      fields["n_layers"] = args.layers
    clk = {}
    r = ref_arm.run_train_steps(fields, micro_batch=args.micro_batch, seq_len=args.seq_len, steps=args.steps,
                                warmup=args.warmup, dtype=dtype, e2e=not args.no_e2e,
                                before_timed=(sampler.start if rank == 0 else None),
                                after_timed=((lambda: clk.update(sampler.stop())) if rank == 0 else None))
    clocks = clk or None
    world = r["world"]
    tokens = world * args.micro_batch * args.seq_len * args.steps
    tok_s = tokens / (r["ms"] / 1e3)
    e2e = None
    if "e2e_ms" in r:
      e2e = {"value": tokens / (r["e2e_ms"] / 1e3), "unit": "tokens/s", "h2d_bytes_per_step": r["h2d_bytes_per_step"],
             "d2h_bytes_per_step": r["d2h_bytes_per_step"], "ms_per_step": r["e2e_ms"] / args.steps}
    flag.finish()
    if rank == 0:
      print(json.dumps({
        "impl": "reference", "metric": "training throughput, Moonlight-16B-A3B (tokens/s whole job; MFU alongside)",
        "value": tok_s, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": r["ms"] / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": dtype, "data": "synthetic uniform-random token ids (.npy shards through the reference's loader), random-init weights",
        "config": {"model": "moonlight-16b-a3b" if not args.layers else f"INVALID-debug-{args.layers}-layers",
                   "global_batch": world * args.micro_batch, "seq_len": args.seq_len,
                   "parallelism": (f"rdep-ep{world}+zero2-dp{world}" if world > 1 else "single-gpu"),
                   "expert_profile": dtype, "activation_checkpoint": "attention (the reference's only mode)",
                   "l2": "per-step working set is far larger than the 126 MB L2"},
        "final_loss": r["final_loss"], "peak_mem_gib": r["peak_mem_gib"], "clocks": clocks, "e2e": e2e,
        "substitutions": ref_env.substitutions(),
        "timed_loop": "nmoe/train.py:88-109 restated around the reference's own objects; logging/checkpoint/eval left out",
      }), flush=True)
    try:
      from nmoe import runtime as ref_runtime
      ref_runtime.finalize()
    except Exception:
      pass
    os._exit(0)
  except BaseException as e:  # noqa: BLE001 - every failure becomes the `unavailable` line
    if isinstance(e, SystemExit):
      raise
    import traceback
    traceback.print_exc(file=sys.stderr)
    flag.fail(f"{type(e).__name__}: {e}" + (f" (world={world_env})" if world_env > 1 else ""))


def main() -> None:
  ap = argparse.ArgumentParser()
  ap.add_argument("--gpus", type=int, default=1)
  ap.add_argument("--steps", type=int, default=5)
  ap.add_argument("--warmup", type=int, default=3)
  ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
  ap.add_argument("--micro-batch", type=int, default=4)
  ap.add_argument("--seq-len", type=int, default=4096)
  ap.add_argument("--layers", type=int, default=None, help="debug only: fewer layers (result is marked invalid)")
  ap.add_argument("--dtype", default=None, choices=["bf16", "fp8", "nvfp4", "nvfp4x16"],
                  help="expert GEMM profile: fp8 = bf16 activations + block-scaled MXFP8 expert GEMMs (the headline configuration)")
  ap.add_argument("--ref-dtype", default="bf16", choices=["bf16", "fp8", "nvfp4"],
                  help="expert profile of the reference arm; its block-scaled profiles need its CuTe-DSL grouped GEMM, "
                       "which only travels to 1-GPU boxes")
  ap.add_argument("--no-e2e", action="store_true")
  ap.add_argument("--config", default=None,
                  help="a model TOML (configs/moonlet_swa.toml, configs/dsv2_slice.toml, ...) instead of the headline "
                       "Moonlight-16B-A3B; its dtype applies unless --dtype is given, batch_size is split over the GPUs")
  ap.add_argument("--zero2-impl", default=None, choices=["fused", "nccl"], help="ZeRO-2 implementation (default: fused peer kernel)")
  ap.add_argument("--capacity-factor", type=float, default=None,
                  help="expert receive buffers as a multiple of the balanced share (rows beyond it are dropped and reported); "
                       "default: lossless buffers, which at N>1 cost one small host read per MoE layer")
  ap.add_argument("--moe-pipeline", action="store_true",
                  help="run the two halves of every MoE layer's tokens on two streams (dispatch / return of one half under the other's GEMMs)")
  ap.add_argument("--overlap-shared", default="auto", choices=["auto", "0", "1"], help="shared-expert MLP on a second stream")
  ap.add_argument("--recompute-h13", action="store_true", help="recompute the experts' up/gate output in backward (saves ~16 GB on one GPU)")
  ap.add_argument("--activation-checkpoint", default="none", choices=["none", "attention", "full"],
                  help="activation recompute policy; 'none' keeps the ~4 GB of attention activations instead of recomputing them")
  args = ap.parse_args()
  if args.dtype is None and args.config is None:
    args.dtype = "fp8"
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
  model_name = "moonlight-16b-a3b"
  if args.config:
    from nmoe_b200.config import from_toml
    over = [f"--activation_checkpoint={args.activation_checkpoint}", f"--moe_save_h13={str(not args.recompute_h13).lower()}",
            f"--moe_overlap_shared={args.overlap_shared}", "--data_path=synthetic"]
    if args.dtype:
      over.append(f"--dtype={args.dtype}")
    if args.layers:
      over.append(f"--n_layers={args.layers}")
    cfg = from_toml(args.config, over, env={})
    args.dtype = cfg.dtype
    args.seq_len = cfg.seq_len
    args.micro_batch = max(1, cfg.batch_size // max(1, world)) if cfg.batch_size >= world else args.micro_batch
    cfg.batch_size = args.micro_batch * world
    model_name = f"{cfg.preset} ({os.path.basename(args.config)})"
  else:
    cfg = moonlight_cfg(world, args.micro_batch, args.seq_len, args.dtype, args.layers, args.activation_checkpoint,
                        not args.recompute_h13, args.overlap_shared)
  if args.zero2_impl:
    cfg.zero2_impl = args.zero2_impl
  if args.capacity_factor is not None:
    cfg.rdep_capacity_factor = args.capacity_factor
  if args.moe_pipeline:
    cfg.moe_pipeline = "true"
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
      "metric": ("training throughput, Moonlight-16B-A3B (tokens/s whole job; MFU alongside)" if not args.config
                 else f"training throughput, {model_name} (tokens/s whole job)"),
      "value": tok_s, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
      "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
      "dtype": args.dtype, "data": "synthetic uniform-random token ids, random-init weights",
      "config": {"model": model_name if args.layers is None else f"INVALID-debug-{args.layers}-layers",
                 "expert_gemms": {"fp8": "block-scaled MXFP8 (E4M3, E8M0 per 32)", "nvfp4": "block-scaled E2M1, E8M0 per 32", "nvfp4x16": "block-scaled NVFP4 (E2M1, UE4M3 per 16, fp32 tensor scale)",
                                  "bf16": "bf16"}.get(args.dtype, args.dtype) + " forward, bf16 backward; bf16 activations",
                 "global_batch": world * mb, "seq_len": S,
                 "parallelism": (f"rdep-ep{world}+zero2-dp{world}" if world > 1 else "single-gpu"),
                 "vocab": cfg.vocab_size, "layers": cfg.n_layers,
                 "experts": f"{cfg.n_routed_experts} top-{cfg.n_activated_experts} + {cfg.n_shared_experts} shared",
                 "activation_checkpoint": args.activation_checkpoint, "moe_save_h13": not args.recompute_h13,
                 "rdep_capacity_factor": cfg.rdep_capacity_factor,
                 "rdep_rows": (trainer.model.rdep.rows_mode if (trainer.model.rdep is not None and trainer.model.rdep.trim_rows) else "fixed"),
                 "moe_pipeline": bool(trainer.model.rdep is not None and trainer.model.rdep.halves is not None), "zero2_overlap": bool(getattr(trainer.opt.dense, "overlap", False)),
                 "l2": "per-step working set (32 GB of weights) is far larger than the 126 MB L2"},
      "tflops_per_gpu": tflops_per_gpu,
      "mfu_vs_nominal_2250": tflops_per_gpu / 2250.0,
      "mfu_vs_measured_sustained": (tflops_per_gpu / peaks["bf16_tflops_sustained"]) if peaks else None,
      "final_loss": final_loss, "peak_mem_gib": peak_alloc, "clocks": clocks, "e2e": e2e,
      "gpu_launches": launches, "zero2_impl": trainer.opt.dense.impl,
    }
    print(json.dumps(out))
  if trainer.model.rdep is not None:
    trainer.model.rdep.close()
  runtime.finalize()


if __name__ == "__main__":
  main()
