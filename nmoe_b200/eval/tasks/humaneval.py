"""HumanEval: complete a function body; correctness = the hidden unit tests pass in the sandbox."""
from ..execution import humaneval_check

STOP = ("\ndef ", "\nclass ", "\nif __name__", "\nprint(", "\n#")


def build_prompt(prompt: str) -> str:
  return prompt


def truncate(completion: str) -> str:
  cut = len(completion)
  for s in STOP:
    i = completion.find(s)
    if i != -1:
      cut = min(cut, i)
  return completion[:cut]


def is_correct(completion: str, meta: dict, prompt: str) -> bool:
  return humaneval_check(prompt, truncate(completion), meta["test"], meta["entry_point"])
