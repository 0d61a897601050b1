"""ctypes access to ``libnmoe_b200.so``.

Launchers are ``extern "C"`` functions taking raw device pointers and a stream
handle and returning 0 on success (a CUDA error code or a negative argument
error otherwise).  There is no eager fallback on a GPU: if the library is not
built, any CUDA op raises.
"""
from __future__ import annotations

import ctypes
from pathlib import Path
from typing import Optional

import torch

_LIB: Optional[ctypes.CDLL] = None
LIB_PATH = Path(__file__).resolve().parent.parent / "lib" / "libnmoe_b200.so"

# number of launches of this library's kernels since the last reset (bench.py reports it)
LAUNCHES = 0


class NativeLibraryError(RuntimeError):
  pass


def lib() -> ctypes.CDLL:
  global _LIB
  if _LIB is None:
    if not LIB_PATH.exists():
      raise NativeLibraryError(
        f"{LIB_PATH} is missing: run `python -m nmoe_b200._build` (or __graft_entry__.build()) first; "
        "CUDA tensors have no fallback path")
    _LIB = ctypes.CDLL(str(LIB_PATH))
  return _LIB


def available() -> bool:
  return LIB_PATH.exists()


def ptr(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
  return ctypes.c_void_p(0 if t is None else t.data_ptr())


def stream() -> ctypes.c_void_p:
  return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def check(rc: int, what: str, n_launch: int = 1) -> None:
  global LAUNCHES
  if rc != 0:
    if rc > 0:
      raise NativeLibraryError(f"{what}: CUDA error {rc} ({_cuda_error_string(rc)})")
    raise NativeLibraryError(f"{what}: bad argument (code {rc})")
  LAUNCHES += n_launch


def _cuda_error_string(rc: int) -> str:
  try:
    rt = ctypes.CDLL("libcudart.so.12")
    rt.cudaGetErrorString.restype = ctypes.c_char_p
    return rt.cudaGetErrorString(rc).decode()
  except OSError:
    return "?"


def reset_launch_count() -> None:
  global LAUNCHES
  LAUNCHES = 0


def launch_count() -> int:
  return LAUNCHES


c_int = ctypes.c_int
c_ll = ctypes.c_longlong
c_float = ctypes.c_float
