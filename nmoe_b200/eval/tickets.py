"""The consumer of evaluation tickets: the other half of ``eval_mode = "k8s_job"``.

The training job's rank 0 saves a model snapshot and drops ``{metrics_dir}/eval_tickets/{run}_{step}.json`` (``eval/hooks.py``)
instead of evaluating on its own GPUs.  This program, run as a long-lived pod or a cron job on a spare GPU, picks the
tickets up and runs the snapshot runner for each:

  python -m nmoe_b200.eval.tickets --dir /data/metrics/eval_tickets [--once] [--poll-s 30] [--keep-snapshots]

A ticket is *claimed* by renaming it to ``*.claimed.{host}-{pid}`` -- atomic on one filesystem, so several consumers can
watch one directory without evaluating a step twice -- and ends as ``*.done`` (with the summary inside) or ``*.failed``
(with the error).  A claim whose owner died is taken over after ``--stale-s`` seconds.  The snapshot directory is deleted
after a successful evaluation unless ``--keep-snapshots`` is given: a Moonlight snapshot is 32 GB.
"""
from __future__ import annotations

import argparse
import json
import os
import shutil
import socket
import subprocess
import sys
import time
from pathlib import Path
from typing import Callable, List, Optional


def pending(directory: Path, stale_s: float = 6 * 3600.0, now: Optional[float] = None) -> List[Path]:
  """Tickets that may be claimed, oldest first: fresh ``*.json`` files and claims nobody has touched for ``stale_s``."""
  now = time.time() if now is None else now
  out = []
  for p in directory.iterdir() if directory.is_dir() else ():
    if p.suffix == ".json":
      out.append(p)
    elif ".claimed." in p.name and now - p.stat().st_mtime > stale_s:
      out.append(p)
  return sorted(out, key=lambda p: (p.stat().st_mtime, p.name))


def claim(ticket: Path, owner: str) -> Optional[Path]:
  """Rename the ticket to this consumer's name.  None when another consumer was faster (the source is gone)."""
  base = ticket.name.split(".json")[0]
  mine = ticket.with_name(f"{base}.json.claimed.{owner}")
  try:
    os.rename(ticket, mine)
  except FileNotFoundError:
    return None
  os.utime(mine, None)               # the claim's age counts from now, not from when the ticket was written
  return mine


def runner_command(t: dict, extra: List[str]) -> List[str]:
  cmd = [sys.executable, "-m", "nmoe_b200.eval.runner", "--snapshot", str(t["snapshot"]), "--run", str(t["run"]), "--step", str(t["step"])]
  if t.get("tasks_file"):
    cmd += ["--tasks-file", str(t["tasks_file"])]
  if t.get("tasks"):
    cmd += ["--tasks", str(t["tasks"])]
  return cmd + list(extra)


def process(ticket: Path, owner: str, *, extra: List[str] = (), keep_snapshots: bool = False, run: Callable = subprocess.run,
            print_fn: Callable = print) -> Optional[str]:
  """Claim and evaluate one ticket.  Returns "done", "failed", or None when the ticket was taken by someone else."""
  mine = claim(ticket, owner)
  if mine is None:
    return None
  base = mine.name.split(".json")[0]
  try:
    t = json.loads(mine.read_text())
    r = run(runner_command(t, list(extra)), capture_output=True, text=True)
    if r.returncode != 0:
      raise RuntimeError(f"runner exited {r.returncode}: {(r.stderr or '')[-800:]}")
    summary = Path(t["snapshot"]) / "summary.json"
    t["summary"] = json.loads(summary.read_text()) if summary.exists() else None
    t["finished"] = time.time()
    mine.write_text(json.dumps(t))
    os.rename(mine, mine.with_name(base + ".json.done"))
    if not keep_snapshots:
      shutil.rmtree(t["snapshot"], ignore_errors=True)
    core = (t["summary"] or {}).get("CORE")
    print_fn(f"[tickets] {t['run']} step {t['step']}: done" + (f", CORE {core:.4f}" if core is not None else ""))
    return "done"
  except Exception as e:             # a broken ticket must not stop the queue
    try:
      mine.write_text(json.dumps({"ticket": base, "error": repr(e), "failed": time.time()}))
      os.rename(mine, mine.with_name(base + ".json.failed"))
    except OSError:
      pass
    print_fn(f"[tickets] {base}: failed: {e}")
    return "failed"


def serve(directory, *, once: bool = False, poll_s: float = 30.0, stale_s: float = 6 * 3600.0, extra: List[str] = (),
          keep_snapshots: bool = False, run: Callable = subprocess.run, sleep: Callable = time.sleep, print_fn: Callable = print,
          max_rounds: Optional[int] = None) -> dict:
  directory = Path(directory)
  owner = f"{socket.gethostname()}-{os.getpid()}"
  counts = {"done": 0, "failed": 0}
  rounds = 0
  while True:
    for t in pending(directory, stale_s):
      res = process(t, owner, extra=extra, keep_snapshots=keep_snapshots, run=run, print_fn=print_fn)
      if res:
        counts[res] += 1
    rounds += 1
    if once or (max_rounds is not None and rounds >= max_rounds):
      return counts
    sleep(poll_s)


def main(argv=None) -> int:
  ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
  ap.add_argument("--dir", required=True, help="{metrics_dir}/eval_tickets of the training job")
  ap.add_argument("--once", action="store_true", help="process what is there and exit (cron); default: keep polling")
  ap.add_argument("--poll-s", type=float, default=30.0); ap.add_argument("--stale-s", type=float, default=6 * 3600.0)
  ap.add_argument("--keep-snapshots", action="store_true")
  ap.add_argument("runner_args", nargs="*", help="after --: extra arguments for the runner, e.g. -- --max-examples 1000")
  a = ap.parse_args(argv)
  c = serve(a.dir, once=a.once, poll_s=a.poll_s, stale_s=a.stale_s, extra=a.runner_args, keep_snapshots=a.keep_snapshots)
  print(json.dumps(c))
  return 0 if not c["failed"] else 1


if __name__ == "__main__":
  raise SystemExit(main())
