"""Batched generation throughput of the serving engine (paged KV cache, continuous batching, MXFP8 expert GEMMs) on a
gpt-oss-20b-shaped model, for comparison with the figures the reference publishes for its own engine on one B200
(nmoe/data/README.md:714-722: gpt-oss-20b 17 tok/s at batch 1, 220 at batch 64, 502 at batch 128).

Weights are random (no checkpoint can be fetched here), which leaves the arithmetic and the memory traffic of every
step unchanged: same layer count, widths, expert count, top-k, GQA ratio, sliding window and vocabulary.  Every
sequence generates exactly ``--new`` tokens (no stop token), prompts are ``--prompt`` random tokens.

  python benchmarks/serve_decode.py --batches 1,64,128 --prompt 128 --new 64

Prints one JSON line per batch size: tokens/s over the whole call (prefill + decode, host scheduling and sampling
included: it is the number a user of ``Engine.generate`` sees) and decode-only tokens/s from CUDA events around the
decode steps.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

PUBLISHED = {"gpt-oss-20b": {1: 17.0, 64: 220.0, 128: 502.0}}     # tok/s, 1 x B200, the reference's README


def main() -> None:
  ap = argparse.ArgumentParser()
  ap.add_argument("--batches", default="1,64,128")
  ap.add_argument("--prompt", type=int, default=128)
  ap.add_argument("--new", type=int, default=64)
  ap.add_argument("--layers", type=int, default=24, help="24 = gpt-oss-20b; fewer only for a quick functional check")
  ap.add_argument("--warmup", type=int, default=1)
  a = ap.parse_args()
  from nmoe_b200.ops import tc_gemm as G
  from nmoe_b200.serve import Engine, ServeConfig, Transformer
  dev = torch.device("cuda")
  cfg = ServeConfig(num_hidden_layers=a.layers)
  batches = [int(b) for b in a.batches.split(",")]
  max_b = max(batches)
  model = Transformer(cfg, dtype=torch.bfloat16, device=dev, max_tokens=max(8192, max_b * a.prompt))
  model.init_weights(std=0.02)
  model.eval()
  n_params = sum(p.numel() for p in model.parameters())
  g = torch.Generator().manual_seed(0)
  for B in batches:
    prompts = [torch.randint(0, cfg.vocab_size, (a.prompt,), generator=g).tolist() for _ in range(B)]
    res = None
    for it in range(a.warmup + 1):
      eng = Engine(model, max_seq_len=a.prompt + a.new + 16, max_batch=B, max_prefill_tokens=max(16384, B * a.prompt))
      # time the decode steps on the device as well: wrap the engine's decode
      ev = []
      inner = eng._decode
      def timed_decode(seqs, _inner=inner, _ev=ev):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        out = _inner(seqs)
        e.record()
        _ev.append((s, e, len(seqs)))
        return out
      eng._decode = timed_decode
      torch.cuda.synchronize()
      t0 = time.perf_counter()
      with torch.inference_mode():
        outs = eng.generate(prompts, max_new_tokens=a.new)
      torch.cuda.synchronize()
      wall = time.perf_counter() - t0
      n_new = sum(len(o) for o in outs)
      dec_ms = sum(s.elapsed_time(e) for s, e, _ in ev)
      dec_tok = sum(n for _, _, n in ev)
      res = {"bench": "serve_decode", "model": "gpt-oss-20b shape, random weights" if a.layers == 24 else f"{a.layers}-layer slice",
             "params_b": round(n_params / 1e9, 2), "batch": B, "prompt_tokens": a.prompt, "new_tokens_per_seq": a.new,
             "generated": n_new, "wall_s": round(wall, 3), "tok_per_s": round(n_new / wall, 1),
             "decode_steps": len(ev), "decode_ms_per_step": round(dec_ms / max(1, len(ev)), 3),
             "decode_tok_per_s_device": round(dec_tok / (dec_ms / 1e3), 1) if dec_ms > 0 else None,
             "prefill_steps": eng.steps["prefill"], "preempted": eng.steps["preempted"]}
      pub = PUBLISHED["gpt-oss-20b"].get(B) if a.layers == 24 else None
      if pub:
        res["reference_published_tok_per_s"] = pub
        res["ratio_to_published"] = round(res["tok_per_s"] / pub, 1)
    G.check_status()
    print(json.dumps(res), flush=True)


if __name__ == "__main__":
  main()
