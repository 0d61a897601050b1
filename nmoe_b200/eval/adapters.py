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


def parse_hf_source(src: str, task: Dict[str, Any]):
  """"hf:<dataset>" with subset / split keys in the task, or the one-string forms "hf:<dataset>:<split>" and
  "hf:<dataset>:<subset>:<split>"."""
  parts = src[3:].split(":")
  if len(parts) == 1:
    return parts[0], task.get("subset"), task.get("split", "validation")
  if len(parts) == 2:
    return parts[0], task.get("subset"), parts[1]
  return parts[0], parts[1], parts[2]


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
      name, subset, split = parse_hf_source(src, task)
      ds = datasets.load_dataset(name, subset, split=split)
    except Exception as e:
      raise RuntimeError(f"task source {src} needs the 'datasets' package and network access: {e}")
    yield from ds
    return
  raise ValueError(f"unknown task source {src!r} (expected jsonl:<path> or hf:<dataset>)")


# Row formats of the multiple-choice sets of the CORE suite that do not fit "question / choices / answer".
# Each returns (prompt text, options, index of the right option).
def _fmt_winogrande(row, task):
  # "The trophy didn't fit the case because _ was too big": the options are the two completed sentences' tails,
  # scored as continuations of the text before the blank plus the candidate
  sent = str(row["sentence"])
  head, _, tail = sent.partition("_")
  return head.rstrip(), [f"{row['option1']}{tail}", f"{row['option2']}{tail}"], int(row["answer"]) - 1


def _fmt_boolq(row, task):
  return f"{row['passage']}\nQuestion: {row['question']}?\nAnswer:", ["no", "yes"], int(bool(row["answer"]))


def _fmt_copa(row, task):
  link = "because" if str(row.get("question", "cause")) == "cause" else "therefore"
  lower = lambda t: t[:1].lower() + t[1:]
  return f"{str(row['premise']).rstrip('.')} {link}", [lower(str(row["choice1"])), lower(str(row["choice2"]))], int(row["label"])


def _fmt_openbookqa(row, task):
  ch = row["choices"]
  return f"Question: {row['question_stem']}\nAnswer:", [str(t) for t in ch["text"]], list(ch["label"]).index(row["answerKey"])


ROW_FORMATS = {"winogrande": _fmt_winogrande, "boolq": _fmt_boolq, "copa": _fmt_copa, "openbookqa": _fmt_openbookqa}


def _choice_of(row: Dict[str, Any], task: Dict[str, Any]):
  fmt = task.get("format")
  if fmt:
    if fmt not in ROW_FORMATS:
      raise ValueError(f"unknown row format {fmt!r}; expected one of {sorted(ROW_FORMATS)}")
    return ROW_FORMATS[fmt](row, task)
  qf, cf, af = task.get("question_field", "question"), task.get("choices_field", "choices"), task.get("answer_field", "answer")
  tmpl = task.get("prompt_template", "Question: {question}\nAnswer:")
  opts = row[cf]
  labels = None
  if isinstance(opts, dict):
    labels = opts.get("label")
    opts = opts.get("text", list(opts.values()))
  ans = row[af]
  if isinstance(ans, str):
    a = ans.strip()
    if labels is not None and a in list(labels):
      ans = list(labels).index(a)                    # ARC mixes "A".."E" and "1".."4" as labels
    else:
      ans = "ABCDEFGH".index(a.upper()) if a.upper() in list("ABCDEFGH") else int(a)
  fields = {k: v for k, v in row.items() if isinstance(v, (str, int, float))}
  fields["question"] = row[qf]
  return tmpl.format(**fields), [str(o) for o in opts], int(ans)


def iter_choices(task: Dict[str, Any], max_examples: Optional[int] = None) -> Iterator[Choice]:
  """Fields (overridable in the task entry): question / choices / answer (index, letter or label), or a named row
  ``format``.  ``fewshot = k`` takes the first k rows as solved examples, joined in front of every later prompt
  (the rows used as shots are not scored)."""
  shots = int(task.get("fewshot", 0))
  prefix: List[str] = []
  n = 0
  for row in _rows(task):
    prompt, opts, ans = _choice_of(row, task)
    if len(prefix) < shots:
      prefix.append(f"{prompt} {opts[ans]}")
      continue
    if max_examples is not None and n >= max_examples:
      return
    n += 1
    yield Choice("\n\n".join(prefix + [prompt]), opts, ans)


def iter_span(task: Dict[str, Any], max_examples: Optional[int] = None) -> Iterator[Span]:
  """Generation examples.  ``format = "squad"`` builds the prompt from context + question and keeps every accepted
  answer in ``meta["answers"]``."""
  pf, rf = task.get("prompt_field", "prompt"), task.get("reference_field", "answer")
  shots = int(task.get("fewshot", 0))
  prefix: List[str] = []
  n = 0
  for row in _rows(task):
    if task.get("format") == "squad":
      answers = row["answers"]["text"] if isinstance(row["answers"], dict) else [a["text"] for a in row["answers"]]
      prompt = f"{row['context']}\nQuestion: {row['question']}\nAnswer:"
      ref, meta = (answers[0] if answers else ""), {"answers": list(answers)}
    else:
      prompt, ref = str(row[pf]), str(row.get(rf, ""))
      meta = {k: v for k, v in row.items() if k not in (pf, rf)}
    if len(prefix) < shots:
      prefix.append(f"{prompt} {ref}")
      continue
    if max_examples is not None and n >= max_examples:
      return
    n += 1
    yield Span("\n\n".join(prefix + [prompt]), ref, meta)
