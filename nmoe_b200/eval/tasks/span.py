"""Extractive question answering scored the SQuAD way: exact match or token F1 after normalisation (lower case,
punctuation and articles removed), best over the accepted answers.  The generated text is cut at the first line
break, since a base model goes on to write the next question."""
from __future__ import annotations

import re
import string
from collections import Counter
from typing import Iterable


def normalize(text: str) -> str:
  text = "".join(ch for ch in text.lower() if ch not in set(string.punctuation))
  text = re.sub(r"\b(a|an|the)\b", " ", text)
  return " ".join(text.split())


def first_line(text: str) -> str:
  text = text.strip()
  return text.split("\n", 1)[0].strip() if text else ""


def f1(pred: str, ref: str) -> float:
  p, r = normalize(pred).split(), normalize(ref).split()
  if not p or not r:
    return float(p == r)
  common = sum((Counter(p) & Counter(r)).values())
  if common == 0:
    return 0.0
  prec, rec = common / len(p), common / len(r)
  return 2 * prec * rec / (prec + rec)


def best_f1(generated: str, answers: Iterable[str]) -> float:
  g = first_line(generated)
  return max((f1(g, a) for a in answers), default=0.0)


def is_correct(generated: str, reference, meta=None) -> bool:
  answers = list((meta or {}).get("answers") or ([reference] if isinstance(reference, str) else list(reference)))
  g = normalize(first_line(generated))
  return any(g == normalize(a) for a in answers)
