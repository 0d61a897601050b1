"""GSM8K: few-shot free-form arithmetic; the answer is the last number of the completion."""
import re

_NUM = re.compile(r"-?\d[\d,]*\.?\d*")


def build_prompt(question: str, shots=()) -> str:
  parts = [f"Question: {q}\nAnswer: {a}\n" for q, a in shots]
  return "\n".join(parts + [f"Question: {question}\nAnswer:"])


def extract_answer(text: str):
  m = re.search(r"####\s*(-?[\d,\.]+)", text)
  s = m.group(1) if m else (_NUM.findall(text.split("Question:")[0]) or [None])[-1]
  if s is None:
    return None
  try:
    return float(s.replace(",", "").rstrip("."))
  except ValueError:
    return None


def is_correct(completion: str, reference: str) -> bool:
  a, b = extract_answer(completion), extract_answer(reference)
  return a is not None and b is not None and abs(a - b) < 1e-6
