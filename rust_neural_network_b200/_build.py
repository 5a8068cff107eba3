"""In-tree build of the native libraries.

Two shared objects are produced next to this file (under ``lib/``):

* ``libb200nn_cuda.so`` - every hand-written sm_100a kernel (plain CUDA, C ABI, no torch headers);
* ``libb200nn_host.so`` - the host runtime in C++ (checkpoint reader/writer, tokenizer, parsers,
  tiered store, TCP store, CPU oracles) with no CUDA dependency, so it loads on a CPU-only machine.

Both are loaded through ``ctypes`` (see ``_native.py``). nvcc cross-compiles for
``compute_100a/sm_100a`` without a GPU being present.
"""
from __future__ import annotations

import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
CSRC = ROOT / "csrc"
LIBDIR = Path(__file__).resolve().parent / "lib"
OBJDIR = ROOT / "build" / "obj"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
]
CXX_FLAGS = ["-O3", "-std=c++17", "-fPIC", "-march=x86-64-v3", "-pthread", "-Wall"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found")


def _digest(path: Path, extra: str) -> str:
    h = hashlib.sha256()
    h.update(extra.encode())
    h.update(path.read_bytes())
    # headers are few: hash them all so that a header edit rebuilds every object
    for hdr in sorted(CSRC.rglob("*.h")) + sorted(CSRC.rglob("*.cuh")):
        h.update(hdr.read_bytes())
    return h.hexdigest()[:16]


def _compile_one(src: Path, cuda: bool, verbose: bool) -> Path:
    flags = NVCC_FLAGS if cuda else CXX_FLAGS
    tag = _digest(src, " ".join(flags))
    obj = OBJDIR / f"{src.stem}.{tag}.o"
    if obj.exists():
        return obj
    for old in OBJDIR.glob(f"{src.stem}.*.o"):
        old.unlink()
    cmd = ([_nvcc()] + NVCC_FLAGS if cuda else [os.environ.get("CXX", "g++")] + CXX_FLAGS) + ["-c", str(src), "-o", str(obj)]
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"compile failed: {src}\n{r.stdout}\n{r.stderr}")
    return obj


def cuda_sources() -> list[Path]:
    return sorted(p for p in CSRC.rglob("*.cu"))


def host_sources() -> list[Path]:
    return sorted(p for p in CSRC.rglob("*.cpp"))


def build_all(verbose: bool = False, jobs: int | None = None) -> dict[str, Path]:
    """Compile every CUDA and C++ source and link the two libraries. Idempotent (content-hashed)."""
    OBJDIR.mkdir(parents=True, exist_ok=True)
    LIBDIR.mkdir(parents=True, exist_ok=True)
    jobs = jobs or max(1, (os.cpu_count() or 2))
    cu, cpp = cuda_sources(), host_sources()
    with cf.ThreadPoolExecutor(max_workers=jobs) as ex:
        cu_futs = [ex.submit(_compile_one, s, True, verbose) for s in cu]
        cpp_futs = [ex.submit(_compile_one, s, False, verbose) for s in cpp]
        cu_objs = [f.result() for f in cu_futs]
        cpp_objs = [f.result() for f in cpp_futs]
    out = {}
    cuda_lib = LIBDIR / "libb200nn_cuda.so"
    # one CUDA runtime per process: link the shared cudart so the kernels use the same runtime instance
    # (current device, streams, lazily loaded modules) as PyTorch, which has it loaded already
    cmd = [_nvcc(), "-shared", "--cudart", "shared", "-o", str(cuda_lib)] + [str(o) for o in cu_objs] + ["-Xcompiler", "-fPIC"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed\n{r.stdout}\n{r.stderr}")
    out["cuda"] = cuda_lib
    if cpp_objs:
        host_lib = LIBDIR / "libb200nn_host.so"
        cmd = [os.environ.get("CXX", "g++"), "-shared", "-o", str(host_lib)] + [str(o) for o in cpp_objs] + ["-pthread"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed\n{r.stdout}\n{r.stderr}")
        out["host"] = host_lib
    return out


if __name__ == "__main__":
    libs = build_all(verbose="-v" in sys.argv)
    for k, v in libs.items():
        print(k, v)
