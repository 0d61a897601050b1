"""Host-side failure detection, as gloo ranks on CPU: a rank that exits or stalls during the peer-handle exchange,
a rank that leaves or stalls between steps.  The survivors must end with an error that names what happened, within
seconds, instead of hanging.  No GPU is involved and nothing is faulted: every failure is made on the host."""
import os
import socket
import subprocess
import sys
import time

import pytest

WORKER = os.path.join(os.path.dirname(os.path.abspath(__file__)), "mp_cpu_worker.py")


def _free_port() -> int:
  with socket.socket() as s:
    s.bind(("127.0.0.1", 0))
    return s.getsockname()[1]


def _run(scenario: str, world: int, limit_s: float = 60.0):
  port = _free_port()
  procs = []
  for r in range(world):
    env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
               GLOO_SOCKET_IFNAME="lo")
    procs.append(subprocess.Popen([sys.executable, WORKER, scenario], env=env, stdout=subprocess.PIPE,
                                  stderr=subprocess.STDOUT, text=True))
  t0 = time.time()
  outs = []
  for p in procs:
    try:
      out, _ = p.communicate(timeout=max(1.0, limit_s - (time.time() - t0)))
    except subprocess.TimeoutExpired:
      p.kill()
      out, _ = p.communicate()
      out += "\nKILLED BY TEST (hang)"
    outs.append(out)
  return outs, time.time() - t0


def test_healthy_exchange_round_trips():
  outs, _ = _run("healthy_exchange", 3)
  assert all("EXCHANGE OK" in o for o in outs), outs


@pytest.mark.parametrize("scenario", ["exit_before_exchange", "stall_in_exchange"])
def test_lost_rank_in_handle_exchange_raises_on_the_others(scenario):
  outs, took = _run(scenario, 2)
  assert "DETECTED exchange" in outs[0] and "KILLED BY TEST" not in outs[0], outs
  assert took < 45, took


def test_rank_that_leaves_between_steps_is_seen_before_the_next_launch():
  outs, took = _run("leave_between_steps", 3)
  for o in outs[:2]:
    assert "DETECTED lost" in o, outs
  # rank 0 hosts the store and can always read why the peer left; rank 1 reads the same unless rank 0 (having raised
  # first) is already gone, in which case it reports the lost store -- also a named PeerLost, not a hang
  assert "injected failure after step 3" in outs[0], outs
  assert "injected failure after step 3" in outs[1] or "store" in outs[1], outs
  assert took < 45, took


def test_rank_that_stalls_between_steps_is_reported():
  outs, took = _run("stall_between_steps", 3)
  assert "DETECTED stalled" in outs[0] and "rank 2" in outs[0], outs
  # rank 1 sees the same stall, unless rank 0 has already raised and taken the store with it (a named PeerLost)
  assert ("DETECTED stalled" in outs[1] and "rank 2" in outs[1]) or ("DETECTED lost" in outs[1] and "store" in outs[1]), outs
  assert took < 45, took


def test_eval_time_budget_is_decided_by_rank_zero_for_all_ranks():
  """Two gloo ranks with different views of the evaluation budget run the same tasks (rank 0's view) and finish."""
  outs, took = _run("eval_budget", 2, limit_s=120.0)
  for o in outs:
    lines = [l for l in o.splitlines() if l.startswith("EVAL TASKS")]
    assert len(lines) == 2 and "KILLED" not in o, o
    assert lines[0] == "EVAL TASKS ['t0', 't1', 't2'] n=[4, 4, 4]" and lines[1] == "EVAL TASKS ['t0']", o


def test_stop_request_is_agreed_on_one_step_by_all_ranks():
  outs, _ = _run("stop_agreement", 3, limit_s=60.0)
  steps = []
  for o in outs:
    line = [l for l in o.splitlines() if l.startswith("STOPPED AT")]
    assert line and "KILLED" not in o, o
    steps.append(line[0])
  assert steps == ["STOPPED AT 6"] * 3, steps          # requested after step 4, margin 2
