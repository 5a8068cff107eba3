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

# warnings are errors in both compilers
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-Wall", "--expt-relaxed-constexpr", "-Werror", "all-warnings",
]
CXX_FLAGS = ["-O3", "-std=c++17", "-fPIC", "-march=x86-64-v3", "-pthread", "-Wall", "-Wextra", "-Werror"]
SANITIZE_FLAGS = ["-O1", "-g", "-fno-omit-frame-pointer", "-fsanitize=address,undefined", "-fno-sanitize-recover=undefined"]


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


def asan_runtime(cxx: str):
    """Absolute path of the compiler's libasan.so, or None when it ships none."""
    r = subprocess.run([cxx, "-print-file-name=libasan.so"], capture_output=True, text=True)
    p = r.stdout.strip()
    return p if r.returncode == 0 and os.path.isabs(p) and os.path.exists(p) else None


def _sanitizer_cxx() -> str:
    for cand in (os.environ.get("CXX"), "g++", "/usr/bin/g++"):
        if cand and shutil.which(cand) and asan_runtime(cand):
            return cand
    raise RuntimeError("no C++ compiler with an AddressSanitizer runtime found")


def build_host_sanitized() -> Path:
    """The host runtime once more with AddressSanitizer + UndefinedBehaviorSanitizer (`lib/libb200nn_host_asan.so`).
    Load it in a process started with LD_PRELOAD=$(g++ -print-file-name=libasan.so) and B200NN_HOST_LIB pointing at it:
    tests/test_cpu_sanitizers.py runs the checkpoint / tokenizer / parser / CPU-kernel tests that way."""
    OBJDIR.mkdir(parents=True, exist_ok=True)
    LIBDIR.mkdir(parents=True, exist_ok=True)
    cxx = _sanitizer_cxx()
    flags = [f for f in CXX_FLAGS if f != "-O3"] + SANITIZE_FLAGS
    objs = []
    for src in host_sources():
        obj = OBJDIR / f"{src.stem}.asan.{_digest(src, ' '.join(flags))}.o"
        if not obj.exists():
            r = subprocess.run([cxx] + flags + ["-c", str(src), "-o", str(obj)], capture_output=True, text=True)
            if r.returncode != 0:
                raise RuntimeError(f"sanitized compile failed: {src}\n{r.stderr}")
        objs.append(obj)
    out = LIBDIR / "libb200nn_host_asan.so"
    r = subprocess.run([cxx, "-shared", "-fsanitize=address,undefined", "-o", str(out)] + [str(o) for o in objs] + ["-pthread"], capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"sanitized link failed\n{r.stderr}")
    return out


def ptxas_report() -> str:
    """Registers, spills, shared memory and stack of every kernel, from `nvcc -Xptxas -v` (no GPU needed). One line per
    kernel: file, demangled kernel name, registers, spill stores / loads, static shared memory, stack frame."""
    import re
    lines = []
    for src in cuda_sources():
        cmd = [_nvcc()] + NVCC_FLAGS + ["-Xptxas", "-v", "-c", str(src), "-o", os.devnull]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"compile failed: {src}\n{r.stderr}")
        name = None
        stack = spill = ""
        for ln in r.stderr.splitlines():
            m = re.search(r"Compiling entry function '(\S+)'", ln)
            if m:
                name = m.group(1)
                continue
            m = re.search(r"(\d+) bytes stack frame, (\d+) bytes spill stores, (\d+) bytes spill loads", ln)
            if m:
                stack, spill = m.group(1), f"{m.group(2)}/{m.group(3)}"
                continue
            m = re.search(r"Used (\d+) registers(?:, used \d+ barriers)?(?:, (\d+) bytes smem)?", ln)
            if m and name:
                dem = subprocess.run(["c++filt", name], capture_output=True, text=True).stdout.strip() or name
                dem = re.sub(r"\(.*", "", dem)
                lines.append(f"{src.relative_to(ROOT)}\t{dem}\tregs={m.group(1)}\tspill(st/ld)={spill or '0/0'}\tsmem={m.group(2) or 0}\tstack={stack or 0}")
                name, stack, spill = None, "", ""
    return "\n".join(lines) + "\n"


if __name__ == "__main__":
    if "--ptxas-report" in sys.argv:
        sys.stdout.write(ptxas_report())
        sys.exit(0)
    if "--sanitize" in sys.argv:
        print(build_host_sanitized())
        sys.exit(0)
    libs = build_all(verbose="-v" in sys.argv)
    for k, v in libs.items():
        print(k, v)
