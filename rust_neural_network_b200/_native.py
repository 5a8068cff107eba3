"""ctypes bindings to the native libraries (see ``_build.py``).

The CUDA library is mandatory on a machine with a GPU: ``cuda()`` raises if it cannot be loaded, so
a GPU run can never silently fall back to eager PyTorch. On a CPU-only machine the package still
imports; ops then use their PyTorch reference implementations (the same ones the tests use as oracles).
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

import torch

LIBDIR = Path(__file__).resolve().parent / "lib"

c_void_p, c_int, c_ll, c_float, c_ull = C.c_void_p, C.c_int, C.c_longlong, C.c_float, C.c_ulonglong


class GemmParams(C.Structure):
    _fields_ = [
        ("M", c_int), ("N", c_int), ("K", c_int), ("batch", c_int), ("splits", c_int),
        ("C", c_void_p), ("ldc", c_ll), ("strideC", c_ll),
        ("bias", c_void_p), ("bias_f32", c_int), ("bias_vec_ok", c_int), ("strideBias", c_ll),
        ("residual", c_void_p), ("ldr", c_ll), ("strideR", c_ll),
        ("aux_out", c_void_p), ("aux_in", c_void_p),
        ("alpha", c_float), ("alpha_ptr", c_void_p), ("act", c_int), ("dact", c_int), ("out_mode", c_int),
        ("vec_ok", c_int), ("res_vec_ok", c_int),
        ("row_scale", c_void_p), ("col_scale", c_void_p),
        ("status", c_void_p),
        ("m_valid", c_void_p), ("k_valid", c_void_p),
    ]


class GemmArgs(C.Structure):
    _fields_ = [
        ("p", GemmParams),
        ("A", c_void_p), ("lda", c_ll), ("strideA", c_ll), ("a_mn", c_int),
        ("B", c_void_p), ("ldb", c_ll), ("strideB", c_ll), ("b_mn", c_int),
        ("M", c_int), ("N", c_int), ("K", c_int), ("batch", c_int), ("dtype", c_int),
    ]


class AttnTensor(C.Structure):
    _fields_ = [("ptr", c_void_p), ("sb", c_ll), ("ss", c_ll), ("sh", c_ll)]


class FlashArgs(C.Structure):
    _fields_ = [
        ("q", AttnTensor), ("k", AttnTensor), ("v", AttnTensor), ("o", AttnTensor),
        ("dout", AttnTensor), ("dq", AttnTensor), ("dk", AttnTensor), ("dv", AttnTensor),
        ("lse", c_void_p), ("delta", c_void_p), ("dq_accum", c_void_p),
        ("B", c_int), ("H", c_int), ("Sq", c_int), ("Skv", c_int), ("hd", c_int),
        ("scale", c_float), ("causal", c_int), ("status", c_void_p),
    ]


_SIGS = {
    # name: argtypes (restype is always int)
    "b200_gemm_launch": [C.POINTER(GemmArgs), c_int, c_int, c_void_p],
    "b200_flash_fwd": [C.POINTER(FlashArgs), c_void_p],
    "b200_flash_bwd": [C.POINTER(FlashArgs), c_void_p],
    "b200_unary": [c_void_p, c_void_p, c_ll, c_int, c_float, c_float, c_int, c_void_p],
    "b200_binary": [c_void_p, c_void_p, c_void_p, c_ll, c_int, c_ll, c_int, c_void_p],
    "b200_cast": [c_void_p, c_void_p, c_ll, c_float, c_int, c_void_p],
    "b200_transpose": [c_void_p, c_void_p, c_int, c_int, c_ll, c_ll, c_ll, c_ll, c_int, c_int, c_void_p],
    "b200_colsum": [c_void_p, c_void_p, c_ll, c_int, c_ll, c_int, c_void_p],
    "b200_dact_colsum": [c_void_p, c_void_p, c_void_p, c_ll, c_int, c_ll, c_ll, c_int, c_void_p],
    "b200_gate": [c_void_p, c_ll, c_void_p, c_ll, c_void_p, c_ll, c_void_p, c_ll, c_void_p, c_ll, c_ll, c_int, c_void_p],
    "b200_colsum_batched": [c_void_p, c_void_p, c_int, c_ll, c_int, c_ll, c_ll, c_int, c_void_p, c_void_p],
    "b200_reduce": [c_void_p, c_void_p, c_ll, c_int, c_int, c_void_p],
    "b200_dropout": [c_void_p, c_void_p, c_ll, c_float, c_ull, c_int, c_void_p],
    "b200_softmax_fwd": [c_void_p, c_void_p, c_ll, c_int, c_float, c_int, c_int, c_void_p],
    "b200_softmax_bwd": [c_void_p, c_void_p, c_void_p, c_ll, c_int, c_float, c_int, c_void_p],
    "b200_fake_quant": [c_void_p, c_void_p, c_ll, c_float, c_float, c_float, c_int, c_void_p],
    "b200_embedding_fwd": [c_void_p, c_void_p, c_void_p, c_ll, c_int, c_ll, c_int, c_void_p],
    "b200_embedding_bwd": [c_void_p, c_void_p, c_void_p, c_ll, c_int, c_ll, c_int, c_void_p],
    "b200_layernorm_fwd": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_ll, c_int, c_float, c_int, c_void_p],
    "b200_add_layernorm_fwd": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_ll, c_int, c_float, c_void_p],
    "b200_layernorm_bwd_sums": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_ll, c_int, c_void_p, c_void_p, c_void_p],
    "b200_layernorm_bwd": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_ll, c_int, c_int, c_void_p],
    "b200_batchnorm_fwd": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_float, c_int, c_int, c_void_p],
    "b200_batchnorm_bwd": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "b200_ce_label": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_ll, c_int, c_ll, c_float, c_float, c_int, c_void_p],
    "b200_ce_dense": [c_void_p, c_void_p, c_void_p, c_void_p, c_ll, c_int, c_float, c_float, c_int, c_void_p],
    "b200_pointwise_loss": [c_void_p, c_void_p, c_void_p, c_void_p, c_ll, c_int, c_float, c_float, c_float, c_int, c_void_p],
    "b200_adam": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_ll, c_float, c_float, c_float, c_float, c_float, c_int, c_void_p, c_void_p, c_void_p],
    "b200_sgd": [c_void_p, c_void_p, c_void_p, c_void_p, c_ll, c_float, c_float, c_void_p, c_void_p, c_void_p],
    "b200_rmsprop": [c_void_p, c_void_p, c_void_p, c_void_p, c_ll, c_float, c_float, c_float, c_void_p, c_void_p],
    "b200_muon_rms": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_float, c_float, c_float, c_void_p],
    "b200_clip_coef": [c_void_p, c_float, c_void_p],
    "b200_incr_step": [c_void_p, c_void_p],
}

_cuda_lib = None
_host_lib = None
_launch_count = 0


def _declare(lib, sigs):
    for name, args in sigs.items():
        try:
            fn = getattr(lib, name)
        except AttributeError:
            continue
        fn.argtypes = args
        fn.restype = c_int


def cuda_available() -> bool:
    return torch.cuda.is_available()


def cuda():
    """Return the CUDA kernel library, loading it on first use. Raises if it is missing."""
    global _cuda_lib
    if _cuda_lib is None:
        path = LIBDIR / "libb200nn_cuda.so"
        if not path.exists():
            raise RuntimeError(
                f"{path} is missing: build it with `python -c 'import __graft_entry__ as g; g.build()'` "
                "(the sm_100a kernels are required on a GPU machine; there is no eager fallback)")
        _cuda_lib = C.CDLL(str(path), mode=C.RTLD_GLOBAL)
        _declare(_cuda_lib, _SIGS)
        _declare(_cuda_lib, _EXTRA_SIGS)
        if torch.cuda.is_available():
            torch.cuda.init()
            # load every tensor-core kernel variant and opt in to its shared-memory carve-out now,
            # from the importing thread, instead of lazily from an autograd worker thread
            for name in ("b200_gemm_init", "b200_flash_fwd_init", "b200_flash_bwd_init", "b200_linattn_init", "b200_gemm_mx_init"):
                fn = getattr(_cuda_lib, name)
                fn.argtypes, fn.restype = [], c_int
                rc = fn()
                if rc != 0:
                    raise RuntimeError(f"{name} failed with CUDA error {rc}")
            if os.environ.get("B200NN_PDL", "1") == "0":
                set_pdl(False)
    return _cuda_lib


_EXTRA_SIGS: dict = {}


def set_pdl(on: bool) -> None:
    """Programmatic dependent launch for the kernels that support it (GEMM, flash attention, LayerNorm, the streaming
    backward helpers): each such kernel may be dispatched, and run its prologue, while its predecessor is still running.
    On by default; `B200NN_PDL=0` in the environment turns it off."""
    lib = _cuda_lib if _cuda_lib is not None else cuda()
    fn = lib.b200_set_pdl
    fn.argtypes, fn.restype = [c_int], c_int
    fn(1 if on else 0)


def set_gemm_pair(on: bool, force: bool = False) -> None:
    """bf16 GEMMs with 256-wide tiles run as 256 x 256 tiles on pairs of CTAs (`cta_group::2`: one MMA across the tensor
    cores of two neighbouring SMs, each staging half of the operands) where that pays: enough pair tiles to fill the
    machine and at least 1024 of K per tile (shorter tiles are bound by their epilogue). On by default;
    `B200NN_GEMM_PAIR=0` in the environment or `set_gemm_pair(False)` keeps single-CTA tiles; `force=True` takes the pair
    kernel for every shape it can run (tests)."""
    lib = _cuda_lib if _cuda_lib is not None else cuda()
    fn = lib.b200_gemm_set_pair
    fn.argtypes, fn.restype = [c_int], c_int
    fn((2 if force else 1) if on else 0)


def set_gemm_tma_store(on: bool) -> None:
    """bf16 GEMM outputs leave the epilogue as TMA stores of 32 x 64 panels (default) or as per-thread 16-byte stores."""
    lib = _cuda_lib if _cuda_lib is not None else cuda()
    fn = lib.b200_gemm_set_tma_store
    fn.argtypes, fn.restype = [c_int], c_int
    fn(1 if on else 0)


def register_sigs(sigs: dict) -> None:
    """Let other modules declare the signatures of kernels they own."""
    _EXTRA_SIGS.update(sigs)
    if _cuda_lib is not None:
        _declare(_cuda_lib, sigs)
    if _host_lib is not None:
        _declare(_host_lib, sigs)


def host():
    """Return the host-side C++ runtime library (no CUDA dependency)."""
    global _host_lib
    if _host_lib is None:
        # B200NN_HOST_LIB selects another build of the host runtime (the sanitizer build of `_build.build_host_sanitized`)
        path = Path(os.environ.get("B200NN_HOST_LIB") or (LIBDIR / "libb200nn_host.so"))
        if not path.exists():
            raise RuntimeError(f"{path} is missing: run the in-tree build first")
        _host_lib = C.CDLL(str(path))
        _declare(_host_lib, _EXTRA_SIGS)
    return _host_lib


def host_available() -> bool:
    return (LIBDIR / "libb200nn_host.so").exists()


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def ptr(t):
    return 0 if t is None else t.data_ptr()


def count_launch(n: int = 1) -> None:
    global _launch_count
    _launch_count += n


def launch_count() -> int:
    return _launch_count


def reset_launch_count() -> None:
    global _launch_count
    _launch_count = 0


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{what} failed with code {rc}")


NVTX_ENABLED = os.environ.get("B200NN_NVTX", "0") == "1"


def traced(family: str):
    """Decorator: run the function inside an NVTX range named after its kernel family when tracing is on
    (`utils.metrics.enable_nvtx()` or B200NN_NVTX=1); one boolean test otherwise."""
    def deco(fn):
        import functools

        @functools.wraps(fn)
        def wrapper(*a, **kw):
            if not NVTX_ENABLED:
                return fn(*a, **kw)
            torch.cuda.nvtx.range_push(family)
            try:
                return fn(*a, **kw)
            finally:
                torch.cuda.nvtx.range_pop()
        return wrapper
    return deco


_status_words: dict = {}


def status_word(device) -> torch.Tensor:
    """Per-device uint32 word that kernels set when a bounded wait expires."""
    key = torch.device(device).index or 0
    if key not in _status_words:
        _status_words[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _status_words[key]


STATUS_NAMES = {
    1: "TMA stage never landed", 2: "TMA stage never released", 3: "accumulator never completed",
    4: "accumulator never drained", 5: "peer flag wait expired", 6: "wait expired", 7: "bad argument / misaligned shared memory",
}


def check_status(device=None) -> None:
    """Synchronise and raise if any kernel recorded a bounded-wait expiry."""
    for key, w in list(_status_words.items()):
        v = int(w.item())
        if v != 0:
            w.zero_()
            raise RuntimeError(f"device kernel reported status {v}: {STATUS_NAMES.get(v, 'unknown')}")
