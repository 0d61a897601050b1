"""Process setup: device selection, seeds, TF32, process group (nmoe/runtime.py:13-77).

One process per GPU; ``RANK`` / ``LOCAL_RANK`` / ``WORLD_SIZE`` / ``MASTER_*`` come from torchrun.
On CUDA the backend is NCCL (plumbing and small all-reduces; the expert and ZeRO-2 hot paths use
peer memory directly), on CPU it is gloo (tests).
"""
from __future__ import annotations

import datetime
import os
from typing import Tuple

import torch
import torch.distributed as dist


def require_b200(device: torch.device) -> None:
  major, minor = torch.cuda.get_device_capability(device)
  if major != 10:
    raise RuntimeError(f"this framework targets sm_100a (B200); device reports compute capability {major}.{minor}")


def init(seed: int = 42, *, device: str = "auto", timeout_s: int = 600) -> Tuple[int, int, torch.device]:
  """Returns (rank, world, device)."""
  rank = int(os.environ.get("RANK", "0"))
  world = int(os.environ.get("WORLD_SIZE", "1"))
  local_rank = int(os.environ.get("LOCAL_RANK", "0"))
  use_cuda = torch.cuda.is_available() if device == "auto" else device == "cuda"
  if use_cuda:
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    require_b200(dev)
    torch.backends.cuda.matmul.allow_tf32 = True
    torch.backends.cudnn.allow_tf32 = True
  else:
    dev = torch.device("cpu")
  torch.manual_seed(seed)
  if use_cuda:
    torch.cuda.manual_seed_all(seed)
  if world > 1 and not dist.is_initialized():
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29500")
    kw = {"device_id": dev} if use_cuda else {}
    dist.init_process_group("nccl" if use_cuda else "gloo", rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=timeout_s), **kw)
  return rank, world, dev


def finalize() -> None:
  if dist.is_initialized():
    try:
      dist.barrier()
    finally:
      dist.destroy_process_group()
