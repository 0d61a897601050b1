"""Make the installed, unmodified reference importable on a box that lacks three of its external dependencies.

``activate()`` puts ``baseline/_ref`` at the front of ``sys.path`` and registers stand-in modules for what the
reference imports but neither ships nor finds on this image.  Nothing under ``baseline/_ref`` is edited, and no
kernel or model of this repository is involved: every stand-in forwards to PyTorch / cuDNN library calls.

===========================  =============================================================  ==========================
module the reference wants    why it is absent                                               stand-in
===========================  =============================================================  ==========================
flash_attn.cute.interface     FlashAttention-4 (CuTe) forward; the reference expects a       cuDNN fused attention
                              checkout under third_party/flash_attn                          through
                              (nmoe/runtime.py:24-32, nmoe/attention/mla.py:69-71)           ``aten::_scaled_dot_
nmoe.csrc.flashmla_sm100      FlashMLA sm100 backward, built from a FlashMLA checkout        product_cudnn_attention``
                              (nmoe/csrc/Makefile:62-74, nmoe/attention/mla.py:72,127)       and its backward
nmoe.blockscaled.grouped      present in the install, but the file names a TMA load with     names that raise when
                              cluster multicast and is therefore left out of snapshots       called; only registered
                              sent to boxes with two or more GPUs                            when the file is absent,
                                                                                             the bf16 profile never
                                                                                             calls them
===========================  =============================================================  ==========================

cuDNN's attention is the fastest library attention for the (192, 128) head dimensions on B200 that this image
offers, so the stand-in does not handicap the reference arm.  ``substitutions()`` lists what was replaced, for the
benchmark's JSON line.
"""
from __future__ import annotations

import importlib
import importlib.util
import os
import sys
import types
from pathlib import Path

HERE = Path(__file__).resolve().parent
REF_ROOT = HERE / "_ref"

_SUBS: list[str] = []
_ACTIVE = False


def substitutions() -> list[str]:
    return list(_SUBS)


class ReferenceUnavailable(RuntimeError):
    pass


# --------------------------------------------------------------------------------------------------------------------
# attention stand-ins (cuDNN through torch)
# --------------------------------------------------------------------------------------------------------------------
_RNG: dict[int, tuple] = {}          # out.data_ptr() -> (philox_seed, philox_offset) of the forward that made it
_BWD_MODE = {"aten": True}


def _equal_length_batch(total: int, cu):
    b = int(cu.numel()) - 1
    if b <= 0 or total % b:
        raise ValueError("stand-in attention supports equal-length packed sequences only")
    return b, total // b


def _fa4_fwd(q, k, v, cu_seqlens_q=None, cu_seqlens_k=None, softmax_scale=None, causal=True, return_lse=True, **_):
    """Same contract as the call in nmoe/attention/mla.py:82-91: q/k [total, H, Dqk], v [total, H, Dv] packed
    equal-length sequences -> (out [total, H, Dv], lse [H, total] fp32)."""
    import torch
    total, h, _dqk = q.shape
    b, s = _equal_length_batch(total, cu_seqlens_q)
    q4 = q.view(b, s, h, -1).transpose(1, 2)
    k4 = k.view(b, s, h, -1).transpose(1, 2)
    v4 = v.view(b, s, h, -1).transpose(1, 2)
    r = torch.ops.aten._scaled_dot_product_cudnn_attention(q4, k4, v4, None, True, 0.0, bool(causal), False,
                                                           scale=float(softmax_scale))
    out4, lse = r[0], r[1]
    out = out4.transpose(1, 2).reshape(total, h, -1)
    if len(_RNG) > 256:
        _RNG.clear()
    _RNG[out.data_ptr()] = (r[6], r[7])
    lse = lse.reshape(b, h, s).permute(1, 0, 2).reshape(h, total).float()
    return out, lse


def _flashmla_dense_prefill_bwd(workspace, d_o, q, k, v, out, lse_t, cu_q, cu_k, dq, dk, dv, causal, softmax_scale,
                                seqlen_q, seqlen_k, is_varlen):
    """Same contract as the call in nmoe/attention/mla.py:127-145: fills dq, dk, dv in place."""
    import torch
    total, h, _ = q.shape
    b, s = _equal_length_batch(total, cu_q)
    q4 = q.view(b, s, h, -1).transpose(1, 2)
    k4 = k.view(b, s, h, -1).transpose(1, 2)
    v4 = v.view(b, s, h, -1).transpose(1, 2)
    do4 = d_o.view(b, s, h, -1).transpose(1, 2)
    g = None
    if _BWD_MODE["aten"]:
        try:
            o4 = out.view(b, s, h, -1).transpose(1, 2)
            lse = lse_t.T.reshape(h, b, s).permute(1, 0, 2).contiguous().view(b, h, s, 1)
            seed, off = _RNG.pop(out.data_ptr(), (None, None))
            if seed is None:
                seed = torch.zeros((), dtype=torch.int64, device=q.device)
                off = torch.zeros((), dtype=torch.int64, device=q.device)
            g = torch.ops.aten._scaled_dot_product_cudnn_attention_backward(
                do4, q4, k4, v4, o4, lse, seed, off, None, None, None, s, s, 0.0, bool(causal),
                scale=float(softmax_scale))
        except Exception as e:  # fall back to autograd through the public SDPA call (one extra forward)
            _BWD_MODE["aten"] = False
            _SUBS.append(f"attention backward stand-in fell back to autograd recompute ({type(e).__name__})")
            g = None
    if g is None:
        from torch.nn.attention import SDPBackend, sdpa_kernel
        with torch.enable_grad(), sdpa_kernel([SDPBackend.CUDNN_ATTENTION, SDPBackend.EFFICIENT_ATTENTION,
                                               SDPBackend.MATH]):
            qa, ka, va = (t.detach().requires_grad_(True) for t in (q4, k4, v4))
            o = torch.nn.functional.scaled_dot_product_attention(qa, ka, va, is_causal=bool(causal),
                                                                 scale=float(softmax_scale))
            g = torch.autograd.grad(o, (qa, ka, va), do4)
    for dst, src in zip((dq, dk, dv), g[:3]):
        dst.copy_(src.transpose(1, 2).reshape(dst.shape))


def _register(name: str, module: types.ModuleType) -> None:
    sys.modules[name] = module
    parent, _, leaf = name.rpartition(".")
    if parent and parent in sys.modules:
        setattr(sys.modules[parent], leaf, module)


def _importable(name: str) -> bool:
    try:
        return importlib.util.find_spec(name) is not None
    except (ImportError, ValueError, AttributeError):
        return False


def activate() -> None:
    """Idempotent.  Raises ReferenceUnavailable naming the one thing that is really missing."""
    global _ACTIVE
    if _ACTIVE:
        return
    if not (REF_ROOT / "nmoe" / "model.py").exists():
        raise ReferenceUnavailable("reference not installed under baseline/_ref (run python baseline/build_ref.py)")
    p = str(REF_ROOT)
    if p in sys.path:
        sys.path.remove(p)
    sys.path.insert(0, p)
    os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")   # as nmoe/train.py:33 does
    # torch first: its bundled cuBLAS / cuBLASLt must be the ones the process binds.  The extension links the
    # toolkit's libcublas by soname; loaded first, it would shadow torch's copy and torch's GEMMs then fail with
    # CUBLAS_STATUS_INVALID_VALUE (seen on the first nn.Linear of the reference model).
    import torch  # noqa: F401
    try:
        importlib.import_module("nmoe.csrc.rdep")
    except Exception as e:
        raise ReferenceUnavailable(f"nmoe.csrc.rdep not importable ({type(e).__name__}: {e}); "
                                   "build it with python baseline/build_ref.py") from e

    # -- FlashAttention-4 CuTe forward
    if not _importable("flash_attn.cute"):
        try:
            importlib.import_module("flash_attn")
        except Exception:
            _register("flash_attn", types.ModuleType("flash_attn"))
        cute = types.ModuleType("flash_attn.cute")
        iface = types.ModuleType("flash_attn.cute.interface")
        iface._flash_attn_fwd = _fa4_fwd
        cute.interface = iface
        _register("flash_attn.cute", cute)
        _register("flash_attn.cute.interface", iface)
        _SUBS.append("flash_attn.cute.interface._flash_attn_fwd (FlashAttention-4, not on this image) -> cuDNN fused "
                     "attention via torch aten::_scaled_dot_product_cudnn_attention")
    # -- FlashMLA sm100 backward
    if not _importable("nmoe.csrc.flashmla_sm100"):
        m = types.ModuleType("nmoe.csrc.flashmla_sm100")
        m.dense_prefill_bwd = _flashmla_dense_prefill_bwd
        _register("nmoe.csrc.flashmla_sm100", m)
        _SUBS.append("nmoe.csrc.flashmla_sm100.dense_prefill_bwd (FlashMLA, sources not in the checkout) -> cuDNN "
                     "fused attention backward via torch")
    # -- the CuTe-DSL grouped GEMM file does not travel to boxes with >= 2 GPUs
    if not (REF_ROOT / "nmoe" / "blockscaled" / "grouped.py").exists():
        importlib.import_module("nmoe.blockscaled") if _importable("nmoe.blockscaled") else None
        g = types.ModuleType("nmoe.blockscaled.grouped")

        def _absent(*_a, **_k):
            raise ReferenceUnavailable("nmoe/blockscaled/grouped.py is not present in this snapshot (it names a "
                                       "cluster-multicast TMA load and is left out of multi-GPU calls); "
                                       "only the reference's bf16 profile can run here")
        for n in ("quantize_weights", "expert_blockscaled", "run_grouped_blockscaled_strided"):
            setattr(g, n, _absent)
        g.QuantizedWeightsFused = type("QuantizedWeightsFused", (), {})
        if "nmoe.blockscaled" not in sys.modules:
            pkg = types.ModuleType("nmoe.blockscaled")
            pkg.__path__ = []  # type: ignore[attr-defined]
            _register("nmoe.blockscaled", pkg)
        _register("nmoe.blockscaled.grouped", g)
        _SUBS.append("nmoe.blockscaled.grouped absent from this snapshot: bf16 expert profile only")
    _ACTIVE = True


def blockscaled_available() -> bool:
    return (REF_ROOT / "nmoe" / "blockscaled" / "grouped.py").exists()
