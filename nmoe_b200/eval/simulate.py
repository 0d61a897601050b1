"""A stand-in for the model under evaluation, for checking the evaluation plumbing without a trained checkpoint.

``SimulatedModel`` answers every example right or wrong by a hash of the example and a seed, so that each kind of task
lands on a chosen accuracy: multiple choice, span extraction, unit-tested code, judged free text
(nmoe/eval/runner.py:43-236 has the same four knobs).  Everything downstream of the model -- task files, adapters,
centred accuracies, the CORE mean, ``summary.json``, the ``eval/*`` metric rows a dashboard reads -- runs as it would
with a real model, which is what a pipeline check before a long training run needs.

Tasks whose source cannot be read here (a Hugging Face dataset without network) fall back to synthetic examples of the
same kind, so the run still covers every task of the file.
"""
from __future__ import annotations

import hashlib
from dataclasses import dataclass
from typing import Any, Dict, Iterator, List, Optional

from .adapters import Choice, Span, iter_choices, iter_span
from .choices import centered_accuracy


@dataclass
class SimConfig:
  acc_choices: float = 0.6       # share of multiple-choice examples answered correctly
  acc_span: float = 0.55         # exact-match rate on span tasks
  acc_unittest: float = 0.5      # pass rate on unit-tested generations
  acc_judge: float = 0.6         # keep rate on judged generations
  seed: int = 123


def _unit(text: str, seed: int) -> float:
  """A number in [0, 1) that depends only on (text, seed)."""
  h = hashlib.blake2b(f"{seed}\x00{text}".encode("utf-8", "replace"), digest_size=8).digest()
  return int.from_bytes(h, "big") / float(1 << 64)


class SimulatedModel:
  def __init__(self, cfg: Optional[SimConfig] = None):
    self.cfg = cfg or SimConfig()

  def choose(self, ex: Choice) -> int:
    r = _unit("C:" + ex.prompt, self.cfg.seed)
    if r < self.cfg.acc_choices or len(ex.options) < 2:
      return ex.answer_idx
    wrong = [i for i in range(len(ex.options)) if i != ex.answer_idx]
    return wrong[int(r * 7919) % len(wrong)]

  def answer(self, ex: Span) -> str:
    if _unit("S:" + ex.prompt, self.cfg.seed) < self.cfg.acc_span:
      return ex.reference
    return "not " + ex.reference[::-1]            # shares no token with the reference

  def passes_tests(self, prompt: str) -> bool:
    return _unit("U:" + prompt, self.cfg.seed) < self.cfg.acc_unittest

  def judged_keep(self, prompt: str) -> bool:
    return _unit("J:" + prompt, self.cfg.seed) < self.cfg.acc_judge


# ---------------------------------------------------------------------------------------------- examples
def synthetic_choices(task: str, n: int, n_options: int = 4) -> Iterator[Choice]:
  for i in range(n):
    yield Choice(f"{task} question {i}: which option is right?", [f"option {chr(65 + j)}" for j in range(n_options)], i % n_options)


def synthetic_spans(task: str, n: int) -> Iterator[Span]:
  for i in range(n):
    yield Span(f"{task} passage {i}: the answer is item{i}. Question: what is the answer?", f"item{i}", {"answers": [f"item{i}"]})


def _examples(kind: str, name: str, task: Dict[str, Any], n: int) -> List[Any]:
  try:
    ex = list((iter_choices if kind == "choices" else iter_span)(task, n))
    if ex:
      return ex
  except Exception:            # no network, no datasets package, missing file: the plumbing check goes on
    pass
  if kind == "choices":
    return list(synthetic_choices(name, n, int(task.get("n_options", 4))))
  return list(synthetic_spans(name, n))


# ---------------------------------------------------------------------------------------------- scoring
def simulate_task(model: SimulatedModel, name: str, task: Dict[str, Any], max_examples: int) -> Dict[str, float]:
  """The result dictionary the real scorers produce (``acc``, ``n``, and ``centered_acc`` / ``f1`` where they apply)."""
  from .tasks import span as span_mod
  kind = task.get("kind", "choices")
  scorer = str(task.get("scorer", "span" if kind != "choices" else "choices"))
  if kind == "choices":
    ex = _examples("choices", name, task, max_examples)
    right = sum(int(model.choose(e) == e.answer_idx) for e in ex)
    opts = sum(len(e.options) for e in ex)
    acc = right / len(ex) if ex else 0.0
    return {"acc": acc, "centered_acc": centered_accuracy(acc, opts / len(ex) if ex else 1.0), "n": float(len(ex))}
  ex = _examples("span", name, task, max_examples)
  if scorer in ("humaneval", "unittest"):
    ok = [model.passes_tests(e.prompt) for e in ex]
    return {"acc": sum(ok) / len(ok) if ok else 0.0, "n": float(len(ok))}
  if scorer == "judge":
    ok = [model.judged_keep(e.prompt) for e in ex]
    return {"acc": sum(ok) / len(ok) if ok else 0.0, "n": float(len(ok))}
  outs = [(model.answer(e), e) for e in ex]
  right = sum(int(span_mod.is_correct(o, e.reference, e.meta)) for o, e in outs)
  f1 = sum(span_mod.best_f1(o, e.meta.get("answers") or [e.reference]) for o, e in outs)
  return {"acc": right / len(ex) if ex else 0.0, "f1": f1 / len(ex) if ex else 0.0, "n": float(len(ex))}


def simulate_suite(tasks: Dict[str, Dict[str, Any]], sim: Optional[SimConfig] = None, max_examples: int = 200) -> Dict[str, Dict[str, float]]:
  model = SimulatedModel(sim)
  return {name: simulate_task(model, name, t, max_examples) for name, t in tasks.items()}
