"""GPQA: four-way multiple choice answered by generating a letter."""
import re


def build_prompt(question: str, options) -> str:
  letters = "ABCD"
  body = "\n".join(f"{letters[i]}. {o}" for i, o in enumerate(options))
  return f"{question}\n{body}\nAnswer with a single letter.\nAnswer:"


def extract_answer(text: str):
  m = re.search(r"\b([ABCD])\b", text.strip().upper())
  return m.group(1) if m else None


def is_correct(completion: str, reference: str) -> bool:
  return extract_answer(completion) == reference.strip().upper()[:1]
