"""CPU (gloo) ranks for the host-side failure-detection tests; launched by test_failure_cpu.py as plain child
processes (RANK / WORLD_SIZE / MASTER_* in the environment).  Every scenario makes its failure on the host: a rank
that exits, never joins, stalls, or raises.  A surviving rank prints ``DETECTED <kind>`` and exits 0."""
import datetime
import os
import sys
import time

import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from nmoe_b200.parallel.health import Health, PeerLost, PeerStalled  # noqa: E402
from nmoe_b200.parallel.peer import PeerExchangeError, exchange_handles  # noqa: E402


def main():
  scenario = sys.argv[1]
  rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
  dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=4))
  t0 = time.time()
  if scenario == "exit_before_exchange":
    if rank == 1:
      os._exit(0)                                  # leaves right after the rendezvous, before the exchange
    try:
      exchange_handles(b"h%d" % rank)
      print("NOT DETECTED", flush=True)
    except PeerExchangeError as e:
      print(f"DETECTED exchange {time.time() - t0:.1f}s {e}", flush=True)
  elif scenario == "stall_in_exchange":
    if rank == 1:
      time.sleep(10)                               # alive, but never reaches the exchange in time
      os._exit(0)
    try:
      exchange_handles(b"h%d" % rank)
      print("NOT DETECTED", flush=True)
    except PeerExchangeError as e:
      print(f"DETECTED exchange {time.time() - t0:.1f}s {e}", flush=True)
  elif scenario == "healthy_exchange":
    got = exchange_handles(b"handle-of-%d" % rank)
    assert got == [b"handle-of-%d" % r for r in range(world)], got
    print("EXCHANGE OK", flush=True)
  elif scenario in ("leave_between_steps", "stall_between_steps"):
    # a loaded test machine can hold a healthy rank up for a second or two: the "leave" scenario must only ever see
    # the loss, and the "stall" scenario's threshold sits well above scheduling noise
    h = Health(rank, world, stall_s=30.0 if scenario == "leave_between_steps" else 4.0)
    dist.barrier()
    try:
      for step in range(1, 200):
        h.check()                                  # before "launching" the step
        time.sleep(0.05)                           # the step
        if rank == world - 1 and step == 3:
          if scenario == "leave_between_steps":
            try:
              raise RuntimeError("injected failure after step 3")
            except RuntimeError as e:
              h.fail(repr(e))                      # what train()'s handler does
              os._exit(1)
          else:
            time.sleep(14)                         # stops making progress, stays alive
            os._exit(0)
        h.beat(step)
      print("NOT DETECTED", flush=True)
    except PeerLost as e:
      print(f"DETECTED lost at step {step} {time.time() - t0:.1f}s {e}", flush=True)
    except PeerStalled as e:
      print(f"DETECTED stalled at step {step} {time.time() - t0:.1f}s {e}", flush=True)
  os._exit(0)                                      # no destroy_process_group: a peer may be gone


if __name__ == "__main__":
  main()
