"""Run untrusted generated Python in a subprocess with a wall-clock limit, limits on address space, CPU time,
file size and process count, and no inherited environment (nmoe/eval/execution.py:37-83).  The program gets its own
session; when it ends or times out the whole process group is killed, so nothing it forked or spawned outlives the
check on the training node.  Used by the HumanEval check."""
from __future__ import annotations

import os
import resource
import signal
import subprocess
import sys
import tempfile
from typing import Tuple


def _limits(mem_bytes: int, cpu_s: int, max_procs: int, max_file_bytes: int):
  def fn():
    resource.setrlimit(resource.RLIMIT_AS, (mem_bytes, mem_bytes))
    resource.setrlimit(resource.RLIMIT_CORE, (0, 0))
    resource.setrlimit(resource.RLIMIT_CPU, (cpu_s, cpu_s + 1))
    resource.setrlimit(resource.RLIMIT_FSIZE, (max_file_bytes, max_file_bytes))
    try:
      resource.setrlimit(resource.RLIMIT_NPROC, (max_procs, max_procs))
    except (ValueError, OSError):
      pass                        # a hard limit below ours is already in force
    os.setsid()
  return fn


def _kill_group(pid: int) -> None:
  try:
    os.killpg(pid, signal.SIGKILL)
  except (ProcessLookupError, PermissionError):
    pass


def run_python(code: str, timeout_s: float = 10.0, mem_mb: int = 1024, max_procs: int = 64,
               max_file_mb: int = 16) -> Tuple[bool, str]:
  """(passed, output tail).  passed = exit code 0 within the time limit."""
  with tempfile.TemporaryDirectory() as d:
    path = os.path.join(d, "prog.py")
    with open(path, "w") as f:
      f.write(code)
    p = subprocess.Popen([sys.executable, "-I", path], cwd=d, env={"PATH": "/usr/bin:/bin"}, stdout=subprocess.PIPE,
                         stderr=subprocess.STDOUT, text=True,
                         preexec_fn=_limits(mem_mb << 20, int(timeout_s) + 1, max_procs, max_file_mb << 20))
    try:
      out, _ = p.communicate(timeout=timeout_s)
      return p.returncode == 0, (out or "")[-2000:]
    except subprocess.TimeoutExpired:
      return False, "timeout"
    finally:
      _kill_group(p.pid)          # the session leader's pid is the group id: children and grandchildren go too
      try:
        p.communicate(timeout=2)
      except Exception:
        pass


def humaneval_check(prompt: str, completion: str, test: str, entry_point: str, timeout_s: float = 10.0) -> bool:
  prog = f"{prompt}{completion}\n\n{test}\n\ncheck({entry_point})\n"
  return run_python(prog, timeout_s)[0]
