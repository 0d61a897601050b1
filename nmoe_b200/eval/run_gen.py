"""Generation evaluation with lockstep decoding (nmoe/eval/run_gen.py:87-336).

Every rank decodes its own prompt but all ranks run the same number of forward passes per step
(no KV cache: the whole prefix is re-run, as in the reference) so that MoE expert parallelism stays
matched.  The next token comes from a chunked-vocabulary argmax / top-k, never from full logits."""
from __future__ import annotations

import argparse
import math
from typing import Any, Dict, List, Optional

import torch
import torch.distributed as dist

from ..data.transforms import get_tokenizer
from ..models.transformer import LOGIT_SCALE
from .adapters import iter_span
from .tasks import REGISTRY


@torch.no_grad()
def argmax_vocab_chunked(h: torch.Tensor, w: torch.Tensor, chunk: int = 32768) -> torch.Tensor:
  best_v = torch.full((h.size(0),), float("-inf"), device=h.device)
  best_i = torch.zeros(h.size(0), dtype=torch.long, device=h.device)
  for s in range(0, w.size(0), chunk):
    v, i = ((h.float() @ w[s:s + chunk].float().t()) * LOGIT_SCALE).max(-1)
    upd = v > best_v
    best_v = torch.where(upd, v, best_v)
    best_i = torch.where(upd, i + s, best_i)
  return best_i


@torch.no_grad()
def topk_vocab_chunked(h: torch.Tensor, w: torch.Tensor, k: int, chunk: int = 32768):
  vals = idxs = None
  for s in range(0, w.size(0), chunk):
    lg = (h.float() @ w[s:s + chunk].float().t()) * LOGIT_SCALE
    v, i = lg.topk(min(k, lg.size(-1)), dim=-1)
    i = i + s
    if vals is None:
      vals, idxs = v, i
    else:
      cv, ci = torch.cat((vals, v), -1), torch.cat((idxs, i), -1)
      vals, sel = cv.topk(k, dim=-1)
      idxs = ci.gather(-1, sel)
  return vals, idxs


@torch.no_grad()
def generate_lockstep(model, prompt_ids: List[int], *, max_new: int, eos_id: int, steps_global: int,
                      temperature: float = 0.0, top_k: int = 0, active: bool = True, pad_multiple: int = 64) -> List[int]:
  """Decodes up to ``max_new`` tokens but always runs ``steps_global`` forwards (dummy once finished)."""
  dev = next(model.parameters()).device
  ids = list(prompt_ids)
  out: List[int] = []
  done = not active
  for _ in range(steps_global):
    L = len(ids)
    pad_to = ((L + pad_multiple - 1) // pad_multiple) * pad_multiple
    tokens = torch.tensor([ids + [eos_id] * (pad_to - L)], dtype=torch.long, device=dev)
    h = model.hidden(tokens)[0, L - 1:L]
    if done:
      continue
    w = model.lm_head.detach()
    if temperature <= 0.0:
      nxt = int(argmax_vocab_chunked(h, w).item())
    else:
      v, i = topk_vocab_chunked(h, w, max(1, top_k or 50))
      p = torch.softmax(v / temperature, -1)
      nxt = int(i[0, torch.multinomial(p[0], 1)].item())
    if nxt == eos_id or len(out) >= max_new:
      done = True
      continue
    out.append(nxt)
    ids.append(nxt)
  return out


@torch.no_grad()
def eval_gen_task(model, enc, name: str, task: Dict[str, Any], *, rank: int, world: int, max_examples: int, eos_id: int,
                  max_new: int = 256) -> Dict[str, float]:
  mod = REGISTRY[task.get("scorer", name)]
  examples = list(iter_span(task, max_examples))
  mine = examples[rank::world]
  per_rank = math.ceil(len(examples) / world) if examples else 0
  was_training = model.training
  model.eval()
  correct = n = 0
  f1_sum = 0.0
  for i in range(per_rank):
    ex = mine[i] if i < len(mine) else examples[0]
    toks = generate_lockstep(model, enc.encode_ordinary(ex.prompt), max_new=max_new, eos_id=eos_id, steps_global=max_new,
                             active=i < len(mine))
    if i < len(mine):
      text = enc.decode(toks)
      if mod is REGISTRY["humaneval"]:
        ok = mod.is_correct(text, ex.meta, ex.prompt)
      elif mod is REGISTRY["span"]:
        ok = mod.is_correct(text, ex.reference, ex.meta)
        f1_sum += mod.best_f1(text, ex.meta.get("answers") or [ex.reference])
      else:
        ok = mod.is_correct(text, ex.reference)
      correct += int(ok)
      n += 1
  t = torch.tensor([correct, n, f1_sum], dtype=torch.float64, device=next(model.parameters()).device)
  if dist.is_initialized() and world > 1:
    dist.all_reduce(t)
  if was_training:
    model.train()
  c, n, f = t.tolist()
  out = {"acc": c / n if n else 0.0, "n": n}
  if mod is REGISTRY["span"]:
    out["f1"] = f / n if n else 0.0
  return out


def main(argv=None) -> None:
  ap = argparse.ArgumentParser(description="generation evals (gsm8k / gpqa / humaneval) on a checkpointed model")
  ap.add_argument("config"); ap.add_argument("--tasks-file", required=True); ap.add_argument("--max-examples", type=int, default=100)
  ap.add_argument("--max-new", type=int, default=256)
  a = ap.parse_args(argv)
  from .. import runtime
  from ..checkpoint import Checkpointer, load_checkpoint
  from ..config import from_toml
  from ..train import Trainer
  cfg = from_toml(a.config)
  rank, world, dev = runtime.init(cfg.seed)
  tr = Trainer(cfg, rank=rank, world=world, device=dev)
  load_checkpoint(Checkpointer(cfg.checkpoint_dir, async_io=False), tr, None, None, cfg, rank)
  from ..config import load_toml
  tasks = {k: v for k, v in load_toml(a.tasks_file).get("tasks", {}).items() if v.get("kind") in ("gen", "span")}
  enc = get_tokenizer(cfg.tokenizer)
  for name, t in tasks.items():
    r = eval_gen_task(tr.model, enc, name, t, rank=rank, world=world, max_examples=a.max_examples, eos_id=cfg.eos_token_id,
                      max_new=a.max_new)
    if rank == 0:
      print(f"{name}: acc={r['acc']:.3f} n={int(r['n'])}")
  runtime.finalize()


if __name__ == "__main__":
  main()
