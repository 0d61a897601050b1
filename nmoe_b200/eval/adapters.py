"""Task adapters: turn a task description (``configs/eval/tasks.toml`` entry) into examples.

Two example kinds: ``Choice(prompt, options, answer_idx)`` for log-likelihood scoring and
``Span(prompt, reference, meta)`` for generation.  Sources: local JSONL files (always) or
HuggingFace datasets (needs ``datasets`` + network; nmoe/eval/adapters.py:35-260)."""
from __future__ import annotations

import json
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Dict, Iterator, List, Optional


@dataclass
class Choice:
  prompt: str
  options: List[str]
  answer_idx: int


@dataclass
class Span:
  prompt: str
  reference: str
  meta: Dict[str, Any] = field(default_factory=dict)


def _rows(task: Dict[str, Any]) -> Iterator[Dict[str, Any]]:
  src = task.get("source", "")
  if src.startswith("jsonl:") or src.endswith(".jsonl"):
    path = Path(src.split(":", 1)[1] if src.startswith("jsonl:") else src)
    with open(path, "r", encoding="utf-8") as f:
      for line in f:
        if line.strip():
          yield json.loads(line)
    return
  if src.startswith("hf:"):
    try:
      import datasets
      name = src[3:]
      ds = datasets.load_dataset(name, task.get("subset"), split=task.get("split", "validation"))
    except Exception as e:
      raise RuntimeError(f"task source {src} needs the 'datasets' package and network access: {e}")
    yield from ds
    return
  raise ValueError(f"unknown task source {src!r} (expected jsonl:<path> or hf:<dataset>)")


def iter_choices(task: Dict[str, Any], max_examples: Optional[int] = None) -> Iterator[Choice]:
  """Fields (overridable in the task entry): question / choices / answer (index or letter)."""
  qf, cf, af = task.get("question_field", "question"), task.get("choices_field", "choices"), task.get("answer_field", "answer")
  tmpl = task.get("prompt_template", "Question: {question}\nAnswer:")
  for n, row in enumerate(_rows(task)):
    if max_examples is not None and n >= max_examples:
      return
    opts = row[cf]
    if isinstance(opts, dict):
      opts = opts.get("text", list(opts.values()))
    ans = row[af]
    if isinstance(ans, str):
      ans = "ABCDEFGH".index(ans.strip().upper()) if ans.strip().upper() in list("ABCDEFGH") else int(ans)
    fields = {k: v for k, v in row.items() if isinstance(v, (str, int, float))}
    fields["question"] = row[qf]
    yield Choice(tmpl.format(**fields), [str(o) for o in opts], int(ans))


def iter_span(task: Dict[str, Any], max_examples: Optional[int] = None) -> Iterator[Span]:
  pf, rf = task.get("prompt_field", "prompt"), task.get("reference_field", "answer")
  for n, row in enumerate(_rows(task)):
    if max_examples is not None and n >= max_examples:
      return
    yield Span(str(row[pf]), str(row.get(rf, "")), {k: v for k, v in row.items() if k not in (pf, rf)})
