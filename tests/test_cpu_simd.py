"""simd.py on CPU, one test per behaviour of rust-nn src/simd.rs:447-580 (the elementwise entry points are thin fronts
of the elementwise kernels on a GPU and of torch on the host; the contract - shapes, in-place `out`, edge cases - is the
reference's)."""
import torch

from rust_neural_network_b200 import simd


def _naive(a, b, m, k, n):
    return (a.view(m, k).double() @ b.view(k, n).double()).float().reshape(-1)


def _rand(n, seed):
    return torch.rand(n, generator=torch.Generator().manual_seed(seed)) * 2 - 1


def test_matmul_matches_naive_small_medium_large():
    for (m, k, n), seed in (((3, 4, 5), 1), ((32, 48, 40), 2), ((130, 257, 190), 3)):   # the last spans the reference's blocks
        a, b, c = _rand(m * k, seed), _rand(k * n, seed + 10), torch.zeros(m * n)
        simd.simd_matmul(a, b, c, m, k, n)
        assert torch.allclose(c, _naive(a, b, m, k, n), atol=1e-3), (m, k, n)


def test_matmul_identity():
    n = 9
    a = _rand(n * n, 4)
    c = torch.zeros(n * n)
    simd.simd_matmul(a, torch.eye(n).reshape(-1), c, n, n, n)
    assert torch.allclose(c, a, atol=1e-6)


def test_matmul_edge_cases():
    c = torch.zeros(1)
    simd.simd_matmul(torch.tensor([3.0]), torch.tensor([4.0]), c, 1, 1, 1)
    assert abs(float(c[0]) - 12.0) < 1e-6
    cz = torch.empty(0)
    simd.simd_matmul(torch.empty(0), torch.empty(0), cz, 0, 0, 0)
    assert cz.numel() == 0


def test_add_mul_relu_scale_write_into_out():
    a = torch.arange(1.0, 10.0)
    b = a * 10
    out = torch.zeros(9)
    assert simd.simd_add(a, b, out) is out and out.tolist() == [11.0, 22.0, 33.0, 44.0, 55.0, 66.0, 77.0, 88.0, 99.0]
    out8 = torch.zeros(8)
    simd.simd_mul(torch.arange(1.0, 9.0), torch.full((8,), 2.0), out8)
    assert out8.tolist() == [2.0, 4.0, 6.0, 8.0, 10.0, 12.0, 14.0, 16.0]
    x = torch.tensor([-2.0, -1.0, 0.0, 1.0, 2.0, -0.5, 0.5, 3.0, -4.0])
    simd.simd_relu(x, out)
    assert out.tolist() == [0.0, 0.0, 0.0, 1.0, 2.0, 0.0, 0.5, 3.0, 0.0]
    simd.simd_scale(torch.arange(1.0, 9.0), 0.5, out8)
    assert out8.tolist() == [0.5, 1.0, 1.5, 2.0, 2.5, 3.0, 3.5, 4.0]


def test_sum_and_features():
    assert abs(float(simd.simd_sum(torch.arange(1.0, 101.0))) - 5050.0) < 1e-2
    assert isinstance(simd.simd_features(), str) and simd.simd_features()
