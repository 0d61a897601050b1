"""The allocation-free RMSNorm backward (``nmoe_rmsnorm_bwd_noalloc``), called through its exported C
symbol the way a host that cannot allocate would call it, must give what the ordinary entry point
gives -- twice in a row, because both calls reuse the same built-in scratch."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _run(fn_name, dy, x, w, rstd, with_scratch):
  from nmoe_b200.ops import _lib as L
  lib = L.lib()
  M, H = x.shape
  dx = torch.empty_like(x)
  dw = torch.empty_like(w)
  st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
  fn = getattr(lib, fn_name)
  fn.restype = ctypes.c_int
  if with_scratch:
    nb = lib.nmoe_rmsnorm_bwd_blocks(M)
    scratch = torch.empty(nb * H, dtype=torch.float32, device=x.device)
    rc = fn(L.ptr(dy), L.ptr(x), L.ptr(w), L.ptr(rstd), L.ptr(dx), L.ptr(dw), L.ptr(scratch), M, H, 0, st)
  else:
    rc = fn(L.ptr(dy), L.ptr(x), L.ptr(w), L.ptr(rstd), L.ptr(dx), L.ptr(dw), M, H, 0, st)
  assert rc == 0, rc
  torch.cuda.synchronize()
  return dx, dw


def test_noalloc_matches_regular_entry_point_twice():
  torch.manual_seed(0)
  dev = torch.device("cuda")
  for call, (M, H) in enumerate([(777, 2048), (64, 512)]):      # second call: smaller, stale scratch present
    x = torch.randn(M, H, device=dev).bfloat16()
    w = (1 + 0.1 * torch.randn(H, device=dev)).bfloat16()
    dy = torch.randn(M, H, device=dev).bfloat16()
    rstd = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-5)
    dx_ref, dw_ref = _run("nmoe_rmsnorm_bwd", dy, x, w, rstd, True)
    before = torch.cuda.memory_allocated()
    dx, dw = _run("nmoe_rmsnorm_bwd_noalloc", dy, x, w, rstd, False)
    # only the two outputs (allocated by this test, the caller) may have appeared
    assert torch.cuda.memory_allocated() - before <= dx.numel() * 2 + dw.numel() * 2 + 1024
    rel = lambda a, b: ((a.float() - b.float()).abs().max() / (b.float().abs().max() + 1e-6)).item()
    assert rel(dx, dx_ref) < 2e-2 and rel(dw, dw_ref) < 2e-2, f"call {call}"
    assert torch.equal(dx, dx_ref) and torch.equal(dw, dw_ref), "same kernels, same order: bit-identical"


def test_noalloc_reaches_the_end_of_the_built_in_scratch():
  """The largest supported width with enough rows that every partial row of the array is used, and a look at the
  driver's own free-memory figure: the caching allocator cannot see an allocation made by a library, the driver can."""
  torch.manual_seed(1)
  dev = torch.device("cuda")
  M, H = 16384, 4096
  x = torch.randn(M, H, device=dev).bfloat16()
  w = (1 + 0.1 * torch.randn(H, device=dev)).bfloat16()
  dy = torch.randn(M, H, device=dev).bfloat16()
  rstd = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-5)
  dx_ref, dw_ref = _run("nmoe_rmsnorm_bwd", dy, x, w, rstd, True)
  _run("nmoe_rmsnorm_bwd_noalloc", dy, x, w, rstd, False)          # first use on this device may load the module
  from nmoe_b200.ops import _lib as L
  lib = L.lib()
  dx, dw = torch.empty_like(x), torch.empty_like(w)                # outputs exist before the measured call
  torch.cuda.synchronize()
  free_before, _ = torch.cuda.mem_get_info()
  st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
  rc = lib.nmoe_rmsnorm_bwd_noalloc(L.ptr(dy), L.ptr(x), L.ptr(w), L.ptr(rstd), L.ptr(dx), L.ptr(dw), M, H, 0, st)
  torch.cuda.synchronize()
  free_after, _ = torch.cuda.mem_get_info()
  assert rc == 0
  assert free_before - free_after <= 0, (free_before, free_after)  # the driver handed out nothing during the call
  assert torch.equal(dx, dx_ref) and torch.equal(dw, dw_ref)


def test_noalloc_rejects_oversize():
  from nmoe_b200.ops import _lib as L
  lib = L.lib()
  H = 8192
  x = torch.zeros(8, H, device="cuda", dtype=torch.bfloat16)
  w = torch.ones(H, device="cuda", dtype=torch.bfloat16)
  rstd = torch.ones(8, device="cuda")
  st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
  rc = lib.nmoe_rmsnorm_bwd_noalloc(L.ptr(x), L.ptr(x), L.ptr(w), L.ptr(rstd), L.ptr(x.clone()), L.ptr(w.clone()),
                                    8, H, 0, st)
  assert rc == -1
