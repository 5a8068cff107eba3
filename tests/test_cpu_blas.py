"""BLAS surface (blas.py) on CPU, one test per behaviour the reference pins (rust-nn src/blas.rs:1195-1700): the four
transpose combinations against a naive triple loop, alpha / beta accumulation, a shape that spans several cache blocks
of the reference, empty and 1 x 1 edges, the convenience wrapper, GEMV in both orientations, the level-1 routines, the
backend object, and the three Strassen cases (even, odd rectangular, below the recursion threshold)."""
import pytest
import torch

from rust_neural_network_b200 import blas
from rust_neural_network_b200.blas import Transpose as T


def _naive(ta, tb, m, n, k, alpha, a, lda, b, ldb, beta, c, ldc):
    out = c.clone()
    for i in range(m):
        for j in range(n):
            acc = 0.0
            for p in range(k):
                av = a[p * lda + i] if ta.is_trans() else a[i * lda + p]
                bv = b[j * ldb + p] if tb.is_trans() else b[p * ldb + j]
                acc += float(av) * float(bv)
            out[i * ldc + j] = alpha * acc + beta * float(c[i * ldc + j])
    return out


def _rand(n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.rand(n, generator=g) * 2 - 1


@pytest.mark.parametrize("ta,tb", [(T.NoTrans, T.NoTrans), (T.NoTrans, T.Trans), (T.Trans, T.NoTrans), (T.Trans, T.Trans)])
def test_sgemm_matches_naive_in_every_orientation(ta, tb):
    m, n, k = 7, 5, 9
    lda = (m if ta.is_trans() else k) + 2            # padded leading dimensions, as a sub-matrix would have
    ldb = (k if tb.is_trans() else n) + 1
    ldc = n + 3
    a = _rand((k if ta.is_trans() else m) * lda, 1)
    b = _rand((n if tb.is_trans() else k) * ldb, 2)
    c = _rand(m * ldc, 3)
    want = _naive(ta, tb, m, n, k, 1.0, a, lda, b, ldb, 0.0, c, ldc)
    got = c.clone()
    blas.sgemm(ta, tb, m, n, k, 1.0, a, lda, b, ldb, 0.0, got, ldc)
    for i in range(m):
        assert torch.allclose(got[i * ldc:i * ldc + n], want[i * ldc:i * ldc + n], atol=1e-5)
        assert torch.equal(got[i * ldc + n:(i + 1) * ldc], c[i * ldc + n:(i + 1) * ldc])      # the padding columns are not touched


def test_sgemm_alpha_beta_accumulation():
    m, n, k = 4, 6, 5
    a, b, c = _rand(m * k, 4), _rand(k * n, 5), _rand(m * n, 6)
    want = _naive(T.NoTrans, T.NoTrans, m, n, k, 2.5, a, k, b, n, -0.75, c, n)
    blas.sgemm(T.NoTrans, T.NoTrans, m, n, k, 2.5, a, k, b, n, -0.75, c, n)
    assert torch.allclose(c, want, atol=1e-5)
    c1 = torch.ones(m * n)
    blas.sgemm(T.NoTrans, T.NoTrans, m, n, k, 0.0, a, k, b, n, 3.0, c1, n)                   # alpha = 0: only the scaling of C
    assert torch.allclose(c1, torch.full((m * n,), 3.0))


def test_sgemm_large_shape_spanning_several_blocks():
    m, n, k = 150, 300, 270                            # more than one MC / NC / KC block of the reference's packed kernel
    a, b = _rand(m * k, 7), _rand(k * n, 8)
    c = torch.zeros(m * n)
    blas.sgemm(T.NoTrans, T.NoTrans, m, n, k, 1.0, a, k, b, n, 0.0, c, n)
    want = a.view(m, k).double() @ b.view(k, n).double()
    assert torch.allclose(c.view(m, n).double(), want, atol=1e-3)


def test_sgemm_zero_and_small_edges():
    c = torch.full((4,), 7.0)
    blas.sgemm(T.NoTrans, T.NoTrans, 2, 2, 0, 1.0, torch.empty(0), 0, torch.empty(0), 0, 0.0, c, 2)
    assert c.tolist() == [0.0, 0.0, 0.0, 0.0]          # k = 0 with beta = 0 clears C
    c = torch.zeros(1)
    blas.sgemm(T.NoTrans, T.NoTrans, 1, 1, 1, 1.0, torch.tensor([3.0]), 1, torch.tensor([4.0]), 1, 0.0, c, 1)
    assert abs(float(c[0]) - 12.0) < 1e-6
    c = torch.full((3,), 5.0)
    blas.sgemm(T.NoTrans, T.NoTrans, 0, 3, 2, 1.0, torch.empty(0), 2, torch.ones(6), 3, 0.0, c, 3)   # m = 0: nothing happens
    assert c.tolist() == [5.0, 5.0, 5.0]
    with pytest.raises(ValueError):
        blas.sgemm(T.NoTrans, T.NoTrans, 2, 2, 2, 1.0, torch.ones(3), 2, torch.ones(4), 2, 0.0, torch.zeros(4), 2)   # A too small


def test_matmul_convenience():
    c = torch.zeros(4)
    blas.matmul(torch.tensor([1.0, 2, 3, 4]), torch.tensor([5.0, 6, 7, 8]), c, 2, 2, 2)
    assert c.tolist() == [19.0, 22.0, 43.0, 50.0]


def test_sgemv_notrans_and_trans():
    a = torch.tensor([1.0, 2, 3, 4, 5, 6])               # [3, 2]
    y = torch.zeros(3)
    blas.sgemv(T.NoTrans, 3, 2, 1.0, a, 2, torch.tensor([1.0, 1.0]), 1, 0.0, y, 1)
    assert y.tolist() == [3.0, 7.0, 11.0]
    yt = torch.zeros(2)
    blas.sgemv(T.Trans, 3, 2, 1.0, a, 2, torch.tensor([1.0, 1.0, 1.0]), 1, 0.0, yt, 1)
    assert yt.tolist() == [9.0, 12.0]
    y2 = torch.tensor([1.0, 0.0, 1.0, 0.0, 1.0, 0.0])    # incy = 2, alpha and beta both in play, x strided too
    blas.sgemv(T.NoTrans, 3, 2, 2.0, a, 2, torch.tensor([1.0, 9.0, 1.0]), 2, 3.0, y2, 2)
    assert y2.tolist() == [9.0, 0.0, 17.0, 0.0, 25.0, 0.0]


def test_level1_routines():
    assert float(blas.sdot(3, torch.tensor([1.0, 2, 3]), 1, torch.tensor([4.0, 5, 6]), 1)) == 32.0
    y = torch.tensor([1.0, 2, 3])
    blas.saxpy(3, 2.0, torch.tensor([10.0, 20, 30]), y)
    assert y.tolist() == [21.0, 42.0, 63.0]
    x = torch.tensor([1.0, 2, 3])
    blas.sscal(3, 2.0, x)
    assert x.tolist() == [2.0, 4.0, 6.0]
    z = torch.zeros(3)
    blas.scopy(3, torch.tensor([7.0, 8, 9]), z)
    assert z.tolist() == [7.0, 8.0, 9.0]
    assert abs(float(blas.snrm2(2, torch.tensor([3.0, 4.0]))) - 5.0) < 1e-5
    assert float(blas.sdot(2, torch.tensor([1.0, 100, 2, 100]), 2, torch.tensor([3.0, 4.0]), 1)) == 11.0      # strided x


def test_backend_object_matches_the_free_function():
    m = n = k = 16
    a, b = _rand(m * k, 9), _rand(k * n, 10)
    c1, c2 = torch.zeros(m * n), torch.zeros(m * n)
    be = blas.NativeBackend()
    be.sgemm(T.NoTrans, T.NoTrans, m, n, k, 1.0, a, k, b, n, 0.0, c1, n)
    blas.sgemm(T.NoTrans, T.NoTrans, m, n, k, 1.0, a, k, b, n, 0.0, c2, n)
    assert float((c1 - c2).abs().max()) < 1e-4
    assert be.name()
    with pytest.raises(NotImplementedError):
        blas.BlasBackend().sgemm(T.NoTrans, T.NoTrans, 1, 1, 1, 1.0, a, 1, b, 1, 0.0, c1, 1)


@pytest.mark.parametrize("m,k,n", [(64, 64, 64), (70, 33, 51), (8, 8, 8)])
def test_strassen_entry_point_matches_the_classical_product(m, k, n):
    """Even square, odd rectangular, and a size below the reference's recursion threshold: the entry point is kept for API
    parity and always returns the classical product (a tensor-core GEMM gains nothing from 7-multiplication recursion)."""
    a, b = _rand(m * k, 11), _rand(k * n, 12)
    c = torch.zeros(m * n)
    blas.gemm_strassen(a, b, c, m, k, n)
    want = a.view(m, k).double() @ b.view(k, n).double()
    assert torch.allclose(c.view(m, n).double(), want, atol=1e-4)
    assert blas.GEMM_STRASSEN_THRESHOLD > 0
