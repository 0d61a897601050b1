"""Weight initialisation that is exact for low-precision parameters.

``torch.nn.init.trunc_normal_`` draws ``uniform(-1, 1)`` in the tensor's own dtype and maps it
through ``erfinv``.  In bf16 the uniform draw rounds to exactly +-1 for roughly one element in a
few hundred, ``erfinv`` returns +-inf there, and the final clamp turns those into the absolute
bounds +-2: a std=0.02 weight matrix ends up sprinkled with 100-sigma outliers (router logits
saturate, routing collapses onto a few experts).  These helpers sample in fp32, truncate, and
then round once to the parameter dtype.
"""
from __future__ import annotations

import torch


@torch.no_grad()
def trunc_normal_(t: torch.Tensor, mean: float = 0.0, std: float = 0.02, a: float = -2.0, b: float = 2.0,
                  generator: torch.Generator | None = None) -> torch.Tensor:
  """In-place N(mean, std) truncated to [a, b] (absolute bounds, the ``torch.nn.init`` convention),
  sampled in fp32 by rejection and written slice by slice along the first dim to bound the scratch."""
  if t.numel() == 0:
    return t
  flat = t.view(t.size(0), -1) if t.dim() > 1 else t.view(1, -1)
  rows = max(1, (64 << 20) // max(1, flat.size(1)))          # <= 64M fp32 elements of scratch at a time
  for r0 in range(0, flat.size(0), rows):
    dst = flat[r0:r0 + rows]
    x = torch.empty(dst.shape, dtype=torch.float32, device=t.device).normal_(mean, std, generator=generator)
    bad = (x < a) | (x > b)
    while bool(bad.any()):                                    # |bound - mean| >> std in practice: almost never taken
      x[bad] = torch.empty(int(bad.sum()), dtype=torch.float32, device=t.device).normal_(mean, std, generator=generator)
      bad = (x < a) | (x > b)
    dst.copy_(x)
  return t


@torch.no_grad()
def normal_(t: torch.Tensor, mean: float = 0.0, std: float = 0.02, generator: torch.Generator | None = None) -> torch.Tensor:
  return trunc_normal_(t, mean, std, float("-inf"), float("inf"), generator)
