"""Dense SwiGLU MLP with the gate and up projections fused into one interleaved weight."""
import torch
from .init import normal_, trunc_normal_
from torch import nn

from .. import ops


class MLP(nn.Module):
  """w13: [2*inter, dim] with row 2j = gate_j and row 2j+1 = up_j; w2: [dim, inter].

  Same math as the reference MLP (nmoe/model.py:34-48): w2(silu(w1 x) * w3 x).
  """

  def __init__(self, dim: int, inter_dim: int, dtype: torch.dtype = torch.bfloat16):
    super().__init__()
    self.dim, self.inter_dim = dim, inter_dim
    self.w13 = nn.Parameter(torch.empty(2 * inter_dim, dim, dtype=dtype))
    self.w2 = nn.Parameter(torch.empty(dim, inter_dim, dtype=dtype))

  def init_weights(self, init_std: float = 0.02) -> None:
    trunc_normal_(self.w13, mean=0.0, std=0.02)
    trunc_normal_(self.w2, mean=0.0, std=init_std)

  def forward(self, x: torch.Tensor) -> torch.Tensor:
    return ops.linear(ops.swiglu(ops.linear(x, self.w13)), self.w2)
