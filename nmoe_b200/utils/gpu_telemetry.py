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


# Bits of NVML's clocks-throttle-reasons mask (public nvml.h).
THROTTLE_APPS = 0x2                    # applications clocks setting
THROTTLE_SW_POWER_CAP = 0x4
THROTTLE_HW_SLOWDOWN = 0x8
THROTTLE_SW_THERMAL = 0x20
THROTTLE_HW_THERMAL = 0x40
THROTTLE_HW_POWER_BRAKE = 0x80


def dashboard_items(snapshot: List[Dict[str, int]]) -> List[tuple]:
  """Metric rows for one telemetry snapshot under the tag names the dashboards read (nmoe/metrics.py:672-719):
  ``gpu/{i}/{utilization_gpu, memory_used_gib, memory_total_gib, power_draw_w, temperature_c, clocks_sm_mhz,
  clocks_sm_max_mhz, throttle_thermal, throttle_power, throttle_hw_slowdown, throttle_apps, ecc_uncorrected}`` and the
  node aggregates ``gpu_agg/{mean_utilization_gpu, total_memory_used_gib, total_power_w, max_temperature_c}``."""
  gib = float(1 << 30)
  items: List[tuple] = []
  util = mem = power = 0.0
  temp = 0.0
  for g in snapshot:
    i, r = int(g["index"]), int(g.get("throttle_reasons", 0))
    row = {
      "utilization_gpu": float(g["util_gpu"]), "utilization_mem": float(g["util_mem"]),
      "memory_used_gib": g["mem_used"] / gib, "memory_total_gib": g["mem_total"] / gib,
      "power_draw_w": g["power_mw"] / 1000.0, "temperature_c": float(g["temp_c"]),
      "clocks_sm_mhz": float(g["sm_clock_mhz"]), "clocks_sm_max_mhz": float(g["sm_clock_max_mhz"]),
      "throttle_thermal": float(bool(r & (THROTTLE_SW_THERMAL | THROTTLE_HW_THERMAL))),
      "throttle_power": float(bool(r & (THROTTLE_SW_POWER_CAP | THROTTLE_HW_POWER_BRAKE))),
      "throttle_hw_slowdown": float(bool(r & THROTTLE_HW_SLOWDOWN)),
      "throttle_apps": float(bool(r & THROTTLE_APPS)),
      "ecc_uncorrected": float(g.get("ecc_uncorrected", 0)),
    }
    items += [(f"gpu/{i}/{k}", v) for k, v in row.items()]
    util += row["utilization_gpu"]
    mem += row["memory_used_gib"]
    power += row["power_draw_w"]
    temp = max(temp, row["temperature_c"])
  if snapshot:
    items += [("gpu_agg/mean_utilization_gpu", util / len(snapshot)), ("gpu_agg/total_memory_used_gib", mem),
              ("gpu_agg/total_power_w", power), ("gpu_agg/max_temperature_c", temp)]
  return items
