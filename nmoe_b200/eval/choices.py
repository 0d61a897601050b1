"""Multiple-choice evaluation by option log-likelihood (nmoe/eval/choices.py:86-345).

All options of one example are scored in ONE forward (a [n_options, T] batch).  The hidden states at
the option positions go through a chunked-vocabulary log-sum-exp, so [T, V] logits are never
materialised.  Ranks take examples round-robin and execute the same number of forwards (ranks that
run out issue a dummy forward) because every MoE forward is a collective across the expert ranks."""
from __future__ import annotations

import argparse
import math
from typing import Any, Dict, List, Optional

import torch
import torch.distributed as dist

from ..config import load_toml
from ..data.transforms import get_tokenizer
from ..models.transformer import LOGIT_SCALE
from .adapters import Choice, iter_choices


def centered_accuracy(acc: float, n_options: float) -> float:
  base = 1.0 / max(1.0, n_options)
  return max(0.0, min(1.0, (acc - base) / (1.0 - base)))


@torch.no_grad()
def logsumexp_vocab_chunked(h: torch.Tensor, w: torch.Tensor, *, logit_scale: float, chunk: int = 32768) -> torch.Tensor:
  """log sum_v exp(scale * h.w_v) for each row of h [N,D] against w [V,D], vocabulary in chunks."""
  out = None
  hf = h.float()
  for s in range(0, w.size(0), chunk):
    lg = (hf @ w[s:s + chunk].float().t()) * logit_scale
    lse = torch.logsumexp(lg, dim=-1)
    out = lse if out is None else torch.logaddexp(out, lse)
  return out


@torch.no_grad()
def score_options(model, enc, ex: Choice, *, pad_to: int, pad_id: int, compute: bool = True) -> List[float]:
  """Sum of log p(option tokens | prompt) per option."""
  dev = next(model.parameters()).device
  p_ids = enc.encode_ordinary(ex.prompt)
  rows, spans = [], []
  for opt in ex.options:
    o_ids = enc.encode_ordinary(" " + opt) or [pad_id]
    full = (p_ids + o_ids)[:pad_to]
    n_opt = max(0, len(full) - len(p_ids))
    spans.append((len(p_ids) - 1, n_opt, o_ids[:n_opt]))
    rows.append(full + [pad_id] * (pad_to - len(full)))
  tokens = torch.tensor(rows, dtype=torch.long, device=dev)
  hidden = model.hidden(tokens)
  if not compute:
    return [float("-inf")] * len(ex.options)
  out = []
  for i, (p0, n, ids) in enumerate(spans):
    if n <= 0 or p0 < 0:
      out.append(float("-inf"))
      continue
    h = hidden[i, p0:p0 + n].float()
    tgt = torch.tensor(ids, dtype=torch.long, device=dev)
    lse = logsumexp_vocab_chunked(h, model.lm_head.detach(), logit_scale=LOGIT_SCALE)
    z = (h * model.lm_head.detach().index_select(0, tgt).float()).sum(-1) * LOGIT_SCALE
    out.append(float((z - lse).sum().item()))
  return out


@torch.no_grad()
def eval_task(model, enc, task: Dict[str, Any], *, rank: int, world: int, max_examples: int, pad_id: int,
              pad_multiple: int = 128, max_len: int = 2048) -> Dict[str, float]:
  was_training = model.training
  model.eval()
  examples = list(iter_choices(task, max_examples))
  mine = examples[rank::world]
  per_rank = math.ceil(len(examples) / world) if examples else 0
  correct = n = opts = 0
  for i in range(per_rank):
    ex = mine[i] if i < len(mine) else (examples[0] if examples else None)
    longest = max(len(enc.encode_ordinary(ex.prompt + " " + o)) for o in ex.options)
    pad_to = min(max_len, ((longest + pad_multiple - 1) // pad_multiple) * pad_multiple)
    scores = score_options(model, enc, ex, pad_to=pad_to, pad_id=pad_id, compute=i < len(mine))
    if i < len(mine):
      n += 1
      opts += len(ex.options)
      correct += int(max(range(len(scores)), key=scores.__getitem__) == ex.answer_idx)
  dev = next(model.parameters()).device
  t = torch.tensor([correct, n, opts], dtype=torch.float64, device=dev)
  if dist.is_initialized() and world > 1:
    dist.all_reduce(t)
  if was_training:
    model.train()
  correct, n, opts = t.tolist()
  acc = correct / n if n else 0.0
  return {"acc": acc, "centered_acc": centered_accuracy(acc, opts / n if n else 1.0), "n": n}


def load_tasks(path: str, which: str = "core") -> Dict[str, Dict[str, Any]]:
  d = load_toml(path)          # expands ${NMOE_*:-default} placeholders (task files point at local copies of the sets)
  tasks = d.get("tasks", d)
  groups = d.get("groups", {})
  if not which or (not groups and which not in tasks):
    names = list(tasks)                      # a file without groups is one group
  elif which in groups:
    names = groups[which]
  elif which in tasks:
    names = [which]                          # a single task by name
  else:
    raise KeyError(f"{path}: no group or task named {which!r}; groups {sorted(groups)}, tasks {sorted(tasks)}")
  return {n: tasks[n] for n in names if n in tasks and tasks[n].get("kind", "choices") == "choices"}


def run_eval(model, cfg, *, rank: int, world: int, max_examples: int = 500, tasks_file: Optional[str] = None,
             group: Optional[str] = None):
  tasks = load_tasks(tasks_file or cfg.eval_tasks_file, group or cfg.eval_tasks)
  enc = get_tokenizer(cfg.tokenizer)
  return {name: eval_task(model, enc, t, rank=rank, world=world, max_examples=max_examples, pad_id=cfg.eos_token_id)
          for name, t in tasks.items()}


def core_metric(res: Dict[str, Dict[str, float]]) -> float:
  """Mean centred accuracy over the tasks (the CORE number when the group is the CORE suite)."""
  return sum(v["centered_acc"] for v in res.values()) / len(res) if res else 0.0


def format_results(res: Dict[str, Dict[str, float]]) -> str:
  return f"mean_centered={core_metric(res):.4f} " + " ".join(f"{k}:acc={v['acc']:.3f}(c={v['centered_acc']:.3f},n={int(v['n'])})" for k, v in res.items())


def main(argv=None) -> None:
  ap = argparse.ArgumentParser(description="score a checkpointed model on multiple-choice tasks")
  ap.add_argument("config"); ap.add_argument("--tasks-file"); ap.add_argument("--max-examples", type=int, default=500)
  ap.add_argument("--group", help="task group of the file (default: the config's eval_tasks)")
  a = ap.parse_args(argv)
  from .. import runtime
  from ..checkpoint import Checkpointer, load_checkpoint
  from ..config import from_toml
  from ..train import Trainer
  cfg = from_toml(a.config)      # left as trained: the checkpoint refuses a configuration with another fingerprint
  rank, world, dev = runtime.init(cfg.seed)
  tr = Trainer(cfg, rank=rank, world=world, device=dev)
  load_checkpoint(Checkpointer(cfg.checkpoint_dir, async_io=False), tr, None, None, cfg, rank)
  res = run_eval(tr.model, cfg, rank=rank, world=world, max_examples=a.max_examples, tasks_file=a.tasks_file, group=a.group)
  if rank == 0:
    print(format_results(res))
  runtime.finalize()


if __name__ == "__main__":
  main()
