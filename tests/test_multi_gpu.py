"""Multi-GPU checks (RDEP over peer memory, fused ZeRO-2, lockstep training) run as child processes,
one rank per GPU.  Skipped when fewer than two GPUs are visible."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least 2 GPUs")
@pytest.mark.parametrize("fused_return", ["1", "0"])
def test_two_rank_rdep_zero2_train(fused_return):
  """Both return paths (GEMM epilogue that stores to the peers / local GEMM + push kernel), with canary areas
  after every peer-visible region."""
  n = 2
  env = dict(os.environ, NMOE_RDEP_FUSED_RETURN=fused_return, NMOE_RDEP_GUARD="4096")
  worker = os.path.join(os.path.dirname(os.path.abspath(__file__)), "mp_worker.py")
  cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
         "--master-addr", "127.0.0.1", "--master-port", "29611", worker]
  r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
  assert r.returncode == 0 and "MP_WORKER_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]
