"""RMSNorm module (weight in the parameter dtype, fp32 statistics)."""
import torch
from torch import nn

from .. import ops


class RMSNorm(nn.Module):
  def __init__(self, dim: int, eps: float = 1e-5, dtype: torch.dtype = torch.bfloat16):
    super().__init__()
    self.dim, self.eps = dim, eps
    self.weight = nn.Parameter(torch.ones(dim, dtype=dtype))

  def forward(self, x: torch.Tensor) -> torch.Tensor:
    return ops.rmsnorm(x, self.weight, self.eps)
