"""Rotary tables with YaRN-style NTK-by-parts scaling (nmoe/attention/rope.py:25-77).

Tables are fp32 [max_len, head_dim/2]; the rotary kernel reads fp32 and rounds once.
"""
import math

import torch
from torch import nn


class RotaryEmbedding(nn.Module):
  def __init__(self, head_dim: int, base: float, initial_context_length: int, max_context_length: int,
               scaling_factor: float = 1.0, ntk_alpha: float = 1.0, ntk_beta: float = 32.0):
    super().__init__()
    freq = base ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim)
    concentration = 1.0
    if scaling_factor > 1.0:
      concentration = 0.1 * math.log(scaling_factor) + 1.0
      d_half = head_dim / 2
      low = d_half * math.log(initial_context_length / (ntk_beta * 2 * math.pi)) / math.log(base)
      high = d_half * math.log(initial_context_length / (ntk_alpha * 2 * math.pi)) / math.log(base)
      if not (0 < low < high < d_half - 1):
        raise ValueError("rope scaling parameters give an empty interpolation ramp")
      ramp = ((torch.arange(int(d_half), dtype=torch.float32) - low) / (high - low)).clamp(0, 1)
      inv_freq = (1.0 / (scaling_factor * freq)) * ramp + (1.0 / freq) * (1 - ramp)
    else:
      inv_freq = 1.0 / freq
    t = torch.arange(max_context_length, dtype=torch.float32)
    ang = torch.outer(t, inv_freq)
    self.register_buffer("cos", ang.cos() * concentration, persistent=False)
    self.register_buffer("sin", ang.sin() * concentration, persistent=False)
