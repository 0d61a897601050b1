"""Install the reference (Noumena-Network/nmoe) and build its compiled extension, unmodified.

Two steps, both offline:

1. ``pip install --no-index --no-build-isolation --target baseline/_ref <reference checkout>`` (pure-Python wheel).
2. Compile the reference's own ``nmoe/csrc/{rdep,quant,ptx,adamw,gemm}.cu`` and ``bindings.cpp -DBUILD_RDEP`` with the
   flags its Makefile uses (``nmoe/csrc/Makefile:32-45``), run the ``-dlink`` step (``:143-147``) and link
   ``baseline/_ref/nmoe/csrc/rdep<EXT_SUFFIX>`` (``:85,146``).  The Makefile itself cannot be used: it aborts when the
   FlashMLA sources are absent (``:72-74``), although nothing in the RDEP extension needs them.  NVSHMEM is left off
   (the Makefile's auto-detection would also leave it off on a box without ``/usr/include/nvshmem_12``).

The sources are copied to a scratch directory first because the reference checkout may be read-only.  Nothing in the
reference is edited.  The result is git-ignored; it is an installation, not product source.

    python baseline/build_ref.py [--reference /path/to/nmoe] [--force]
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
import sysconfig
import tempfile
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
REF_TARGET = HERE / "_ref"
CUDA_SRCS = ("rdep", "quant", "ptx", "adamw", "gemm")


def _default_reference() -> Path:
    """$NMOE_REFERENCE, else a checkout named ``reference`` next to this repository."""
    env = os.environ.get("NMOE_REFERENCE")
    return Path(env) if env else HERE.parent.parent / "reference"


def ext_path() -> Path:
    return REF_TARGET / "nmoe" / "csrc" / ("rdep" + sysconfig.get_config_var("EXT_SUFFIX"))


def _run(cmd: list[str], cwd: Path) -> None:
    r = subprocess.run(cmd, cwd=cwd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"{' '.join(cmd[:3])} ... failed:\n{r.stdout[-4000:]}")


def install_python(reference: Path) -> None:
    """pip-install the reference's Python package into baseline/_ref (from a copy: its tree may be read-only)."""
    if (REF_TARGET / "nmoe" / "train.py").exists():
        return
    with tempfile.TemporaryDirectory() as tmp:
        src = Path(tmp) / "nmoe_src"
        shutil.copytree(reference, src, ignore=shutil.ignore_patterns("build", "*.egg-info", "nviz", ".git"))
        cmd = [sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation", "--no-deps",
               "--find-links", "/opt/wheelhouse", "--target", str(REF_TARGET), str(src)]
        _run(cmd, cwd=Path(tmp))


def build_extension(reference: Path, force: bool = False) -> Path:
    """Compile the reference's RDEP extension with its Makefile's flags; returns the built module's path."""
    out = ext_path()
    if out.exists() and not force:
        return out
    csrc = reference / "nmoe" / "csrc"
    if not csrc.is_dir():
        raise RuntimeError(f"reference sources not found under {csrc}")
    import pybind11

    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    nvcc = os.path.join(cuda_home, "bin", "nvcc")
    nvcc_flags = ["-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-rdc=true",
                  "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-DNMOE_ENABLE_PTX_E2M1=1",
                  f"-I{cuda_home}/include"]
    cxx_flags = ["-std=c++17", "-O3", "-fPIC", f"-I{cuda_home}/include",
                 f"-I{sysconfig.get_path('include')}", f"-I{pybind11.get_include()}"]
    ldflags = ["-shared", f"-L{cuda_home}/lib64", "-lcublas", "-lcublasLt", "-lcudart", "-lcudadevrt",
               f"-Wl,-rpath,{cuda_home}/lib64"]
    with tempfile.TemporaryDirectory() as tmp:
        work = Path(tmp)
        for f in csrc.iterdir():
            if f.suffix in (".cu", ".cuh", ".cpp", ".h"):
                shutil.copy(f, work / f.name)
        jobs = [[nvcc, *nvcc_flags, "-c", f"{s}.cu", "-o", f"{s}.o"] for s in CUDA_SRCS]
        jobs.append(["g++", *cxx_flags, "-DBUILD_RDEP", "-c", "bindings.cpp", "-o", "bindings_rdep.o"])
        with ThreadPoolExecutor(len(jobs)) as pool:
            list(pool.map(lambda c: _run(c, work), jobs))
        objs = [f"{s}.o" for s in CUDA_SRCS]
        _run([nvcc, *nvcc_flags, "-dlink", "-o", "dlink.o", *objs, "-lcudadevrt"], work)
        out.parent.mkdir(parents=True, exist_ok=True)
        _run(["g++", "-o", str(out), *objs, "dlink.o", "bindings_rdep.o", *ldflags], work)
    return out


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--reference", type=Path, default=_default_reference())
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    install_python(a.reference)
    so = build_extension(a.reference, force=a.force)
    print(f"reference installed under {REF_TARGET}; extension {so} ({so.stat().st_size >> 10} KiB)")


if __name__ == "__main__":
    main()
