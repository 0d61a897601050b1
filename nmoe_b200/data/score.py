"""Oracle scoring: ask the grading model for rubric scores as JSON and parse the answer.

The prompt is a chat-formatted conversation (system / developer / user turns rendered by a
``ChatFormat``; the default renders the Harmony layout ``<|start|>role<|message|>...<|end|>``) whose
developer turn holds the rubric and whose user turn holds the (right-trimmed) document.  Completions
are produced by the continuous-batching engine, greedy, until the end-of-turn token or the budget;
the first JSON object in the answer supplies the five rubric scores (code documents use a code
rubric with its own aggregate).

Reference counterpart: nmoe/data/score.py:64-249.
"""
from __future__ import annotations

import json
import re
from dataclasses import dataclass
from typing import Dict, Iterable, List, Optional, Protocol, Sequence

RUBRIC = ("helpfulness", "correctness", "coherence", "complexity", "density")
CODE_RUBRIC = ("correctness", "readability", "documentation", "complexity", "reusability")

RUBRIC_TEXT = (
  "You grade training data. Score the document on each dimension from 0 (worst) to 4 (best):\n"
  "helpfulness: would a learner gain from reading it; correctness: factual and logical accuracy;\n"
  "coherence: structure and flow; complexity: depth of the ideas; density: information per token.\n"
  'Answer with one JSON object: {"helpfulness": n, "correctness": n, "coherence": n, "complexity": n, "density": n}'
)
CODE_RUBRIC_TEXT = (
  "You grade source code used as training data. Score 0 (worst) to 4 (best) on: correctness, readability,\n"
  "documentation, complexity (non-trivial logic), reusability.\n"
  'Answer with one JSON object: {"correctness": n, "readability": n, "documentation": n, "complexity": n, "reusability": n}'
)


class Tokenizer(Protocol):
  def encode(self, text: str) -> List[int]: ...
  def decode(self, ids: Sequence[int]) -> str: ...


class ByteTokenizer:
  """UTF-8 bytes as tokens (ids 0..255) plus a few control ids; lets the pipeline run without a vocabulary file."""
  eot = 256

  def encode(self, text: str) -> List[int]:
    return list(text.encode("utf-8"))

  def decode(self, ids: Sequence[int]) -> str:
    return bytes(i for i in ids if 0 <= i < 256).decode("utf-8", errors="replace")


@dataclass
class ChatFormat:
  """Renders role-tagged turns to text; ``stop`` are the token ids that end the assistant turn."""
  start: str = "<|start|>"
  message: str = "<|message|>"
  end: str = "<|end|>"

  def render(self, turns: Sequence[tuple]) -> str:
    body = "".join(f"{self.start}{role}{self.message}{text}{self.end}" for role, text in turns)
    return body + f"{self.start}assistant{self.message}"


def build_prompt(tok: Tokenizer, text: str, *, is_code: bool = False, fmt: Optional[ChatFormat] = None) -> List[int]:
  fmt = fmt or ChatFormat()
  turns = [("system", "Reasoning: low"), ("developer", CODE_RUBRIC_TEXT if is_code else RUBRIC_TEXT), ("user", text)]
  return tok.encode(fmt.render(turns))


def right_trim(tok: Tokenizer, text: str, *, is_code: bool = False, max_ctx: int = 4096, max_new: int = 256,
               fmt: Optional[ChatFormat] = None) -> List[int]:
  """Prompt for ``text`` cut (from the right end of the document) so that prompt + answer fit in ``max_ctx``."""
  ids = build_prompt(tok, text, is_code=is_code, fmt=fmt)
  room = max_ctx - max_new
  if len(ids) <= room:
    return ids
  over = len(ids) - room
  doc = tok.encode(text)
  keep = max(0, len(doc) - over - 8)
  return build_prompt(tok, tok.decode(doc[:keep]), is_code=is_code, fmt=fmt)[:room]


_JSON = re.compile(r"\{[^{}]*\}", re.S)


def parse_scores(answer: str, *, is_code: bool = False) -> Optional[Dict[str, float]]:
  """First JSON object in ``answer`` that has every rubric key with a number in [0, 4]; else None."""
  keys = CODE_RUBRIC if is_code else RUBRIC
  for m in _JSON.finditer(answer):
    try:
      j = json.loads(m.group(0))
    except ValueError:
      continue
    try:
      out = {k: float(j[k]) for k in keys}
    except (KeyError, TypeError, ValueError):
      continue
    if all(0.0 <= v <= 4.0 for v in out.values()):
      return out
  return None


def compute_aggregated(scores: Dict[str, float]) -> float:
  """Mean of the five scores mapped to [0, 1] (nmoe/data/score.py:225-238)."""
  vals = [min(max(float(scores[k]) / 4.0, 0.0), 1.0) for k in RUBRIC if k in scores]
  return sum(vals) / len(vals) if vals else 0.0


def compute_aggregated_code(scores: Dict[str, float]) -> float:
  """Code rubric: correctness counts double."""
  w = {"correctness": 2.0, "readability": 1.0, "documentation": 1.0, "complexity": 1.0, "reusability": 1.0}
  num = sum(min(max(float(scores[k]) / 4.0, 0.0), 1.0) * w[k] for k in CODE_RUBRIC if k in scores)
  den = sum(w[k] for k in CODE_RUBRIC if k in scores)
  return num / den if den > 0 else 0.0


def grade_prompts(engine, tok: Tokenizer, texts: Sequence[str], *, is_code: Optional[Sequence[bool]] = None,
                  max_new: int = 256, max_ctx: int = 4096, stop_tokens: Iterable[int] = (),
                  fmt: Optional[ChatFormat] = None) -> List[dict]:
  """Rows ``{scores, aggregated, raw}`` in input order; ``scores`` is None when no valid JSON came back."""
  code = list(is_code) if is_code is not None else [False] * len(texts)
  prompts = [right_trim(tok, t, is_code=c, max_ctx=max_ctx, max_new=max_new, fmt=fmt) for t, c in zip(texts, code)]
  outs = engine.generate(prompts, max_new_tokens=max_new, stop_tokens=stop_tokens)
  rows = []
  for o, c in zip(outs, code):
    raw = tok.decode(o)
    s = parse_scores(raw, is_code=c)
    agg = (compute_aggregated_code(s) if c else compute_aggregated(s)) if s else None
    rows.append({"scores": s, "aggregated": agg, "raw": raw})
  return rows
