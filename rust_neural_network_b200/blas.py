"""BLAS surface of the reference (rust-nn src/blas.rs): `Transpose`, `sgemm`, `sgemv`, `sdot`, `saxpy`,
`sscal`, `scopy`, `snrm2`, `matmul`, `gemm_strassen`, backed by this package's kernels.

`sgemm` is the tcgen05 GEMM: operands may be fp32 (run as TF32 on the tensor cores, fp32
accumulate) or bf16; transposes are folded into the TMA / matrix descriptors exactly as the
reference folds them into packing (src/blas.rs:104-186). beta != 0 uses the kernel's fp32
accumulate path. `sgemv` is the bandwidth-bound GEMV kernel, the level-1 routines are small
grid-stride kernels. Arguments are torch tensors (flat or shaped) instead of slices; outputs are
written in place into `c` / `y` and also returned.

`gemm_strassen` keeps the reference's contract (C = A B, opt-in) but runs the classical
tensor-core product: Strassen trades multiplications for additions and extra memory traffic,
which is a loss on hardware whose multiply throughput dwarfs its bandwidth (src/blas.rs:846-879
notes the same caveat for accuracy).
"""
from __future__ import annotations

import ctypes as C
import enum

import torch

from . import _native as nv
from .ops import gemm as G

_P, _LL, _I, _F = C.c_void_p, C.c_longlong, C.c_int, C.c_float
nv.register_sigs({
    "b200_gemv": [_P, _I, _LL, _I, _P, _P, _I, _I, _F, _F, _P],
    "b200_dot": [_P, _LL, _P, _LL, _LL, _P, _I, _P],
    "b200_axpy": [_F, _P, _P, _LL, _P],
    "b200_scal": [_F, _P, _LL, _P],
})


class Transpose(enum.Enum):
    NoTrans = 0
    Trans = 1

    def is_trans(self) -> bool:
        return self is Transpose.Trans


def _view2d(t: torch.Tensor, rows: int, cols: int, ld: int) -> torch.Tensor:
    """[rows, cols] view with leading dimension `ld` of a flat (or already 2-D) buffer."""
    flat = t.reshape(-1)
    need = (rows - 1) * ld + cols if rows > 0 else 0
    if flat.numel() < need:
        raise ValueError(f"buffer of {flat.numel()} elements is too small for {rows}x{cols} with ld {ld}")
    return torch.as_strided(flat, (rows, cols), (ld, 1))


def sgemm(transa: Transpose, transb: Transpose, m: int, n: int, k: int, alpha: float, a: torch.Tensor, lda: int,
          b: torch.Tensor, ldb: int, beta: float, c: torch.Tensor, ldc: int) -> torch.Tensor:
    """C[m, n] = alpha * op(A) op(B) + beta * C (row-major, leading dimensions as in the reference)."""
    if m == 0 or n == 0:
        return c
    cv = _view2d(c, m, n, ldc)
    if k == 0 or alpha == 0.0:
        cv.mul_(beta) if beta != 0.0 else cv.zero_()
        return c
    # the kernel's contract is C = A' B'^T with A' logical [m, k], B' logical [n, k]
    A = _view2d(a, k, m, lda) if transa.is_trans() else _view2d(a, m, k, lda)          # stored [k, m] -> MN-major
    B = _view2d(b, n, k, ldb) if transb.is_trans() else _view2d(b, k, n, ldb)          # stored [k, n] -> MN-major
    a_mn, b_mn = transa.is_trans(), not transb.is_trans()
    if beta == 0.0:
        out = G.gemm(A, B, a_mn=a_mn, b_mn=b_mn, alpha=alpha, out_dtype=torch.float32)
        cv.copy_(out)
    else:
        if beta != 1.0:
            cv.mul_(beta)
        if c.dtype == torch.float32 and cv.is_contiguous() and c.is_cuda:
            G.gemm(A, B, a_mn=a_mn, b_mn=b_mn, alpha=alpha, accumulate_into=cv)
        else:
            cv.add_(G.gemm(A, B, a_mn=a_mn, b_mn=b_mn, alpha=alpha, out_dtype=torch.float32).to(cv.dtype))
    return c


def sgemv(trans: Transpose, m: int, k: int, alpha: float, a: torch.Tensor, lda: int, x: torch.Tensor, incx: int, beta: float,
          y: torch.Tensor, incy: int) -> torch.Tensor:
    """y = alpha * op(A) x + beta * y with A [m, k] row-major. NoTrans: y has m entries; Trans: k entries."""
    A = _view2d(a, m, k, lda)
    n_in, n_out = (m, k) if trans.is_trans() else (k, m)
    xv = x.reshape(-1)[: (n_in - 1) * incx + 1: incx] if n_in > 0 else x.reshape(-1)[:0]
    yv = y.reshape(-1)[: (n_out - 1) * incy + 1: incy] if n_out > 0 else y.reshape(-1)[:0]
    if not a.is_cuda:
        Af = A.float()
        r = alpha * ((Af.t() @ xv.float()) if trans.is_trans() else (Af @ xv.float()))
        yv.copy_(r + (beta * yv.float() if beta != 0.0 else 0.0))
        return y
    if A.dtype not in (torch.float32, torch.bfloat16):
        A = A.float()
    xc = xv.float().contiguous()
    yc = yv if (yv.dtype == torch.float32 and yv.is_contiguous()) else yv.float().contiguous()
    nv.check(nv.cuda().b200_gemv(A.data_ptr(), 1 if A.dtype == torch.bfloat16 else 0, A.stride(0), 1 if trans.is_trans() else 0,
                                 xc.data_ptr(), yc.data_ptr(), m, k, float(alpha), float(beta), nv.stream_ptr()), "gemv")
    nv.count_launch(2 if trans.is_trans() else 1)
    if yc is not yv:
        yv.copy_(yc)
    return y


def _dot(x, incx, y, incy, n, sqrt_result):
    if not x.is_cuda:
        xv, yv = x.reshape(-1)[: max((n - 1) * incx + 1, 0): incx].float(), y.reshape(-1)[: max((n - 1) * incy + 1, 0): incy].float()
        r = (xv * yv).sum()
        return r.sqrt() if sqrt_result else r
    xc = x.reshape(-1) if x.dtype == torch.float32 else x.reshape(-1).float()
    yc = y.reshape(-1) if y.dtype == torch.float32 else y.reshape(-1).float()
    out = torch.empty(1, dtype=torch.float32, device=x.device)
    nv.check(nv.cuda().b200_dot(xc.data_ptr(), incx, yc.data_ptr(), incy, n, out.data_ptr(), 1 if sqrt_result else 0, nv.stream_ptr()), "dot")
    nv.count_launch()
    return out[0]


def sdot(n: int, x: torch.Tensor, incx: int, y: torch.Tensor, incy: int) -> torch.Tensor:
    """sum_i x[i incx] y[i incy] as a 0-d device tensor (no host sync)."""
    return _dot(x, incx, y, incy, n, False)


def snrm2(n: int, x: torch.Tensor) -> torch.Tensor:
    return _dot(x, 1, x, 1, n, True)


def saxpy(n: int, alpha: float, x: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
    """y[:n] += alpha * x[:n] in place."""
    if not y.is_cuda or y.dtype != torch.float32 or x.dtype != torch.float32 or not y.is_contiguous() or not x.is_contiguous():
        y.reshape(-1)[:n].add_(x.reshape(-1)[:n].to(y.dtype), alpha=alpha)
        return y
    nv.check(nv.cuda().b200_axpy(float(alpha), x.data_ptr(), y.data_ptr(), n, nv.stream_ptr()), "axpy")
    nv.count_launch()
    return y


def sscal(n: int, alpha: float, x: torch.Tensor) -> torch.Tensor:
    if not x.is_cuda or x.dtype != torch.float32 or not x.is_contiguous():
        x.reshape(-1)[:n].mul_(alpha)
        return x
    nv.check(nv.cuda().b200_scal(float(alpha), x.data_ptr(), n, nv.stream_ptr()), "scal")
    nv.count_launch()
    return x


def scopy(n: int, x: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
    y.reshape(-1)[:n].copy_(x.reshape(-1)[:n])
    return y


def matmul(a: torch.Tensor, b: torch.Tensor, c: torch.Tensor, m: int, k: int, n: int) -> torch.Tensor:
    """C = A B for contiguous [m, k] @ [k, n] -> [m, n]."""
    return sgemm(Transpose.NoTrans, Transpose.NoTrans, m, n, k, 1.0, a, k, b, n, 0.0, c, n)


def gemm_strassen(a: torch.Tensor, b: torch.Tensor, c: torch.Tensor, m: int, k: int, n: int) -> torch.Tensor:
    return matmul(a, b, c, m, k, n)


GEMM_STRASSEN_THRESHOLD = 256      # kept for API parity; the tensor-core product never recurses


class BlasBackend:
    """Pluggable GEMM provider (src/blas.rs:712-734): `name()` and `sgemm(...)`."""

    def name(self) -> str:
        raise NotImplementedError

    def sgemm(self, transa, transb, m, n, k, alpha, a, lda, b, ldb, beta, c, ldc):
        raise NotImplementedError


class NativeBackend(BlasBackend):
    """The built-in provider: the tcgen05 GEMM on CUDA tensors, the fp32 reference on CPU tensors."""

    def name(self) -> str:
        return "native-sm100a-tcgen05" if torch.cuda.is_available() else "native-cpu-reference"

    def sgemm(self, transa, transb, m, n, k, alpha, a, lda, b, ldb, beta, c, ldc):
        return sgemm(transa, transb, m, n, k, alpha, a, lda, b, ldb, beta, c, ldc)



from ._compat import install as _install  # noqa: E402

_install(globals())
