"""In-tree build of the native library.

Every ``csrc/**/*.cu`` / ``*.cpp`` is compiled with nvcc for sm_100a only and linked
into ``nmoe_b200/lib/libnmoe_b200.so``.  The sources include no torch or pybind
headers (the Python side talks to ``extern "C"`` launchers through ctypes), so a
full rebuild takes seconds and cross-compiles on a machine without a GPU.
"""
from __future__ import annotations

import hashlib
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
CSRC = ROOT / "csrc"
LIB_DIR = Path(__file__).resolve().parent / "lib"
OBJ_DIR = LIB_DIR / "obj"
LIB_PATH = LIB_DIR / "libnmoe_b200.so"

NVCC_FLAGS = [
  "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
  "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-I", str(CSRC),
]


def _nvcc() -> str:
  cand = os.environ.get("NVCC") or "/usr/local/cuda/bin/nvcc"
  return cand if Path(cand).exists() else "nvcc"


HYBRID_SRC = CSRC / "hybrid" / "rdep_nvshmem.cu"        # built separately (needs NVSHMEM and relocatable device code)
HYBRID_LIB_PATH = LIB_DIR / "libnmoe_hybrid.so"


def _sources() -> list[Path]:
  return sorted(p for p in CSRC.rglob("*") if p.suffix in (".cu", ".cpp") and p != HYBRID_SRC)


def _headers_digest() -> str:
  h = hashlib.sha256()
  for p in sorted(CSRC.rglob("*")):
    if p.suffix in (".cuh", ".h", ".hpp"):
      h.update(p.read_bytes())
  h.update(" ".join(NVCC_FLAGS).encode())
  return h.hexdigest()


def _compile_one(src: Path, hdr: str, verbose: bool, ptxas_v: bool) -> Path:
  tag = hashlib.sha256(src.read_bytes() + hdr.encode()).hexdigest()[:16]
  rel = src.relative_to(CSRC).as_posix().replace("/", "_")
  obj = OBJ_DIR / f"{rel}.{tag}.o"
  if obj.exists():
    return obj
  for old in OBJ_DIR.glob(f"{rel}.*.o"):
    old.unlink()
  cmd = [_nvcc(), *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
  if src.suffix == ".cpp":
    cmd.insert(1, "-x")
    cmd.insert(2, "cu")
  if ptxas_v:
    cmd += ["-Xptxas", "-v"]
  if verbose:
    print(" ".join(cmd), flush=True)
  r = subprocess.run(cmd, capture_output=True, text=True)
  if r.returncode != 0:
    raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
  if ptxas_v:
    print(r.stderr)
  return obj


def build(verbose: bool = False, ptxas_v: bool = False, force: bool = False) -> Path:
  """Compile what changed and relink.  Returns the path of the shared library."""
  OBJ_DIR.mkdir(parents=True, exist_ok=True)
  if force:
    for o in OBJ_DIR.glob("*.o"):
      o.unlink()
  hdr = _headers_digest()
  srcs = _sources()
  if not srcs:
    raise RuntimeError(f"no sources under {CSRC}")
  with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
    objs = list(ex.map(lambda s: _compile_one(s, hdr, verbose, ptxas_v), srcs))
  stamp = LIB_DIR / "link.stamp"
  want = " ".join(o.name for o in objs)
  if LIB_PATH.exists() and stamp.exists() and stamp.read_text() == want:
    return LIB_PATH
  cmd = [_nvcc(), "-shared", "-o", str(LIB_PATH), *map(str, objs), "-lcudart", "-ldl", "-lpthread",
         "-gencode", "arch=compute_100a,code=sm_100a"]
  if verbose:
    print(" ".join(cmd), flush=True)
  r = subprocess.run(cmd, capture_output=True, text=True)
  if r.returncode != 0:
    raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
  stamp.write_text(want)
  return LIB_PATH


def nvshmem_home() -> Path | None:
  """Root of an NVSHMEM installation with include/nvshmem.h and lib/libnvshmem_device.a: $NVSHMEM_HOME, the
  nvidia-nvshmem-cu12 wheel, or the distribution's /usr paths."""
  cands = []
  if os.environ.get("NVSHMEM_HOME"):
    cands.append(Path(os.environ["NVSHMEM_HOME"]))
  try:
    import nvidia.nvshmem as _n  # type: ignore
    cands += [Path(p) for p in _n.__path__]
  except Exception:
    pass
  cands.append(Path("/usr/local/nvshmem"))
  for c in cands:
    if (c / "include" / "nvshmem.h").exists() and (c / "lib" / "libnvshmem_device.a").exists():
      return c
  return None


def build_hybrid(verbose: bool = False) -> Path | None:
  """Build the NVSHMEM-backed inter-node transport (csrc/hybrid/rdep_nvshmem.cu) into lib/libnmoe_hybrid.so.
  Returns None when no NVSHMEM installation is found.  Steps: compile with relocatable device code, device-link
  against libnvshmem_device.a, link the host side against libnvshmem_host."""
  home = nvshmem_home()
  if home is None:
    return None
  OBJ_DIR.mkdir(parents=True, exist_ok=True)
  tag = hashlib.sha256(HYBRID_SRC.read_bytes() + _headers_digest().encode() + str(home).encode()).hexdigest()[:16]
  obj, dobj = OBJ_DIR / f"hybrid_rdep_nvshmem.{tag}.o", OBJ_DIR / f"hybrid_dlink.{tag}.o"
  stamp = LIB_DIR / "hybrid.stamp"
  if HYBRID_LIB_PATH.exists() and stamp.exists() and stamp.read_text() == tag:
    return HYBRID_LIB_PATH
  arch = ["-gencode", "arch=compute_100a,code=sm_100a"]
  cuda_lib = str(Path(_nvcc()).resolve().parent.parent / "lib64") if Path(_nvcc()).exists() else "/usr/local/cuda/lib64"
  host_so = next((p for p in sorted((home / "lib").glob("libnvshmem_host.so*"))), None)
  if host_so is None:
    return None
  steps = [
    [_nvcc(), *arch, "-O3", "-std=c++17", "-rdc=true", "-Xcompiler", "-fPIC", "-I", str(CSRC), "-I", str(home / "include"),
     "-c", str(HYBRID_SRC), "-o", str(obj)],
    [_nvcc(), *arch, "-dlink", "-Xcompiler", "-fPIC", "-o", str(dobj), str(obj), str(home / "lib" / "libnvshmem_device.a"),
     "-lcudadevrt"],
    ["g++", "-shared", "-o", str(HYBRID_LIB_PATH), str(obj), str(dobj), str(home / "lib" / "libnvshmem_device.a"),
     f"-L{home / 'lib'}", f"-l:{host_so.name}", f"-L{cuda_lib}", f"-L{cuda_lib}/stubs", "-lcudadevrt", "-lcudart",
     "-lcuda", f"-Wl,-rpath,{home / 'lib'}", f"-Wl,-rpath,{cuda_lib}"],
  ]
  for cmd in steps:
    if verbose:
      print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
      raise RuntimeError(f"hybrid build step failed: {' '.join(cmd[:4])} ...\n{r.stdout[-3000:]}\n{r.stderr[-3000:]}")
  stamp.write_text(tag)
  return HYBRID_LIB_PATH


if __name__ == "__main__":
  if "--hybrid" in sys.argv:
    print(build_hybrid(verbose="-v" in sys.argv))
    sys.exit(0)
  p = build(verbose="-v" in sys.argv, ptxas_v="--ptxas" in sys.argv, force="--force" in sys.argv)
  print(p)
