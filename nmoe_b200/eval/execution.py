"""Run untrusted generated Python in a subprocess with a wall-clock limit, an address-space limit and
no inherited environment (nmoe/eval/execution.py:37-83).  Used by the HumanEval check."""
from __future__ import annotations

import os
import resource
import subprocess
import sys
import tempfile
from typing import Tuple


def _limits(mem_bytes: int):
  def fn():
    resource.setrlimit(resource.RLIMIT_AS, (mem_bytes, mem_bytes))
    resource.setrlimit(resource.RLIMIT_CORE, (0, 0))
    os.setsid()
  return fn


def run_python(code: str, timeout_s: float = 10.0, mem_mb: int = 1024) -> Tuple[bool, str]:
  """(passed, output tail).  passed = exit code 0 within the time limit."""
  with tempfile.TemporaryDirectory() as d:
    path = os.path.join(d, "prog.py")
    with open(path, "w") as f:
      f.write(code)
    try:
      r = subprocess.run([sys.executable, "-I", path], cwd=d, env={"PATH": "/usr/bin:/bin"}, capture_output=True,
                         text=True, timeout=timeout_s, preexec_fn=_limits(mem_mb << 20))
    except subprocess.TimeoutExpired:
      return False, "timeout"
    return r.returncode == 0, (r.stdout + r.stderr)[-2000:]


def humaneval_check(prompt: str, completion: str, test: str, entry_point: str, timeout_s: float = 10.0) -> bool:
  prog = f"{prompt}{completion}\n\n{test}\n\ncheck({entry_point})\n"
  return run_python(prog, timeout_s)[0]
