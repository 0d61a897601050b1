"""Python face of the native NVML poller (``csrc/telemetry/nvml_poller.cpp``): start / stop /
snapshot (utilisation, memory, power, temperature, SM clock, throttle reasons, ECC).  Read-only."""
from __future__ import annotations

import ctypes
from typing import Dict, List, Optional

from ..ops import _lib as L

_FIELDS = ("index", "util_gpu", "util_mem", "mem_used", "mem_total", "power_mw", "temp_c", "sm_clock_mhz",
           "sm_clock_max_mhz", "throttle_reasons", "ecc_uncorrected", "ts_ms")


class GpuPoller:
  def __init__(self, interval_ms: int = 1000, nvml_path: Optional[str] = None):
    self.interval_ms, self.nvml_path = interval_ms, nvml_path

  def start(self) -> None:
    rc = L.lib().nmoe_gpu_poller_start(self.interval_ms, (self.nvml_path or "").encode())
    if rc != 0:
      raise RuntimeError(f"NVML poller could not start (code {rc})")

  def stop(self) -> None:
    L.lib().nmoe_gpu_poller_stop()

  def is_running(self) -> bool:
    return bool(L.lib().nmoe_gpu_poller_running())

  def snapshot(self, max_gpus: int = 16) -> List[Dict[str, int]]:
    buf = (ctypes.c_int64 * (13 * max_gpus))()
    n = L.lib().nmoe_gpu_poller_snapshot(buf, max_gpus)
    return [{k: int(buf[i * 13 + j]) for j, k in enumerate(_FIELDS)} for i in range(n)]
