"""Elementwise surface of the reference's SIMD module (rust-nn src/simd.rs): `simd_matmul`, `simd_add`,
`simd_mul`, `simd_relu`, `simd_scale`, `simd_sum`, `simd_features`.

The reference's AVX2 loops become this package's vectorised CUDA elementwise / reduction kernels
(16-byte accesses, grid-stride); `simd_matmul` is the tensor-core GEMM. Functions take torch
tensors, write into `out` when one is given (as the reference's `&mut [f32]` output), and return it.
"""
from __future__ import annotations

import torch

from .ops import gemm as G
from .ops import kernels as K


def _finish(r: torch.Tensor, out):
    if out is None:
        return r
    out.reshape(-1)[: r.numel()].copy_(r.reshape(-1))
    return out


def simd_matmul(a: torch.Tensor, b: torch.Tensor, c: torch.Tensor, m: int, k: int, n: int) -> torch.Tensor:
    """C[m, n] = A[m, k] B[k, n] (row-major, contiguous)."""
    r = G.gemm(a.reshape(m, k), b.reshape(k, n), b_mn=True, out_dtype=torch.float32)
    c.reshape(-1)[: m * n].copy_(r.reshape(-1))
    return c


def simd_add(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor = None) -> torch.Tensor:
    return _finish(K.binary(a, b, "add"), out)


def simd_mul(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor = None) -> torch.Tensor:
    return _finish(K.binary(a, b, "mul"), out)


def simd_relu(x: torch.Tensor, out: torch.Tensor = None) -> torch.Tensor:
    return _finish(K.unary(x, "relu"), out)


def simd_scale(x: torch.Tensor, scale: float, out: torch.Tensor = None) -> torch.Tensor:
    return _finish(K.unary(x, "scale", scale), out)


def simd_sum(x: torch.Tensor) -> torch.Tensor:
    """Sum of all elements as a 0-d fp32 tensor on x's device (no host sync)."""
    return K.reduce_all(x, "sum")


def simd_features() -> str:
    """Which vector hardware the kernels of this build target."""
    if torch.cuda.is_available():
        p = torch.cuda.get_device_properties(torch.cuda.current_device())
        return f"CUDA sm_{p.major}{p.minor} ({p.name}): {p.multi_processor_count} SMs, tcgen05 tensor cores, 16-byte vector loads"
    return "CPU reference path (PyTorch); CUDA kernels compiled for sm_100a"


from ._compat import install as _install  # noqa: E402

_install(globals())
