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
  elif scenario == "eval_budget":
    # ranks whose clocks disagree about the evaluation's time budget must still run the same tasks: rank 0 decides
    import json
    import tempfile
    import torch
    from nmoe_b200.config import Config
    from nmoe_b200.eval import runner
    from nmoe_b200.train import Trainer
    d = tempfile.mkdtemp()
    mc = os.path.join(d, "mc.jsonl")
    with open(mc, "w") as f:
      for i in range(4):
        f.write(json.dumps({"question": f"q{i}?", "choices": ["a", "b"], "answer": i % 2}) + "\n")
    tf = os.path.join(d, "tasks.toml")
    with open(tf, "w") as f:
      f.write('[groups]\ncore = ["t0", "t1", "t2"]\n' + "".join(f'[tasks.t{k}]\nkind = "choices"\nsource = "jsonl:{mc}"\n' for k in range(3)))
    cfg = Config(vocab_size=257, eos_token_id=256, tokenizer="bytes", dim=64, n_layers=2, n_heads=2, inter_dim=128, moe_inter_dim=32,
                 n_routed_experts=4, n_activated_experts=2, n_shared_experts=1, n_dense_layers=2, q_lora_rank=32, kv_lora_rank=16,
                 qk_nope_head_dim=16, qk_rope_head_dim=8, v_head_dim=16, batch_size=2, seq_len=64, max_position_embeddings=512,
                 activation_checkpoint="none", metrics_dir=os.path.join(d, "m"), eval_tasks_file=tf, eval_tasks="core")
    torch.manual_seed(0)
    model = Trainer(cfg, rank=rank, world=world).model
    # rank 0 has time for everything, the others think the budget is spent after the first task
    res = runner.run_snapshot_eval(model, cfg, run_id="mp", step=1, max_examples=4, max_time_s=600.0 if rank == 0 else 0.0,
                                   print_fn=lambda *_: None)
    print(f"EVAL TASKS {sorted(res)} n={[int(r['n']) for r in res.values()]}", flush=True)
    res = runner.run_snapshot_eval(model, cfg, run_id="mp", step=2, max_examples=4, max_time_s=0.0 if rank == 0 else 600.0,
                                   print_fn=lambda *_: None)
    print(f"EVAL TASKS {sorted(res)}", flush=True)
  elif scenario == "stop_agreement":
    # three ranks step in lock-step (a barrier stands in for the step's collectives); rank 1 is asked to stop after
    # its step 4.  Every rank must leave at the same step, and that step must lie after the request.
    from nmoe_b200.utils.stop import StopRequest
    stopper = StopRequest(world, install=False)
    left = None
    for step in range(1, 50):
      dist.barrier()
      if rank == 2:
        time.sleep(0.02)                           # one rank lags inside the step
      if rank == 1 and step == 4:
        stopper.request("SIGTERM")
      if stopper.should_stop(step):
        left = step
        break
    print(f"STOPPED AT {left}", flush=True)
  os._exit(0)                                      # no destroy_process_group: a peer may be gone


if __name__ == "__main__":
  main()
