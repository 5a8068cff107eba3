"""int8.py, one test per behaviour of rust-nn src/int8.rs:330-470: per-row symmetric int8 weights, the int8 linear
layer against its fp32 original, and the uint8 x int8 -> int32 product against exact integer arithmetic."""
import pytest
import torch

from rust_neural_network_b200 import nn
from rust_neural_network_b200.int8 import Int8Linear, Int8Weights, igemm, igemm_scalar


def test_round_trip_error_is_small():
    w = torch.tensor([[0.1, 0.2, 0.3, -0.4], [0.5, -0.6, 0.7, 0.8]])
    q = Int8Weights.quantize(w)
    assert q.quantization_error(w) < 0.01
    assert float((q.dequantize() - w).abs().max()) <= 0.8 / 127 / 2 + 1e-7   # half a step of the coarser row


def test_compression_ratio_is_near_four():
    q = Int8Weights.quantize(torch.randn(64, 128))
    assert 3.0 < q.compression_ratio() <= 4.0


def test_memory_is_smaller_than_fp32():
    q = Int8Weights.quantize(torch.randn(32, 64))
    assert q.mem_bytes() == 32 * 64 + 32 * 4
    assert q.mem_bytes() < 32 * 64 * 4


def test_linear_matches_fp32_within_the_quantisation_error():
    torch.manual_seed(0)
    layer = nn.Linear(8, 4)
    x = torch.randn(2, 8)
    want = layer(x).detach()
    got = Int8Linear.from_linear(layer).forward(x)
    assert tuple(got.shape) == (2, 4)
    assert float((got.float() - want).abs().max()) < 0.1


def test_weights_shape():
    q = Int8Weights.quantize(torch.randn(16, 32))
    assert q.shape == [16, 32] and q.data.numel() == 16 * 32 and q.scales.numel() == 16
    assert q.data.dtype == torch.int8


def test_igemm_known_small():
    a = torch.tensor([1, 2, 3, 4], dtype=torch.uint8)
    b = torch.tensor([1, -1, 2, 2, -3, 4, 0, -2], dtype=torch.int8)           # [4, 2]
    assert igemm(a, b, 1, 4, 2).reshape(-1).tolist() == [-4, 7]


def _lcg(seed, n, signed):
    out = []
    for _ in range(n):
        seed = (seed * 1664525 + 1013904223) & 0xFFFFFFFF
        v = (seed >> 16) & 0xFF
        out.append((v - 256 if v >= 128 else v) if signed else (v & 0x7F))
    return seed, out


@pytest.mark.parametrize("m,k,n", [(16, 32, 48), (3, 5, 7), (13, 17, 29), (1, 1, 1), (4, 4, 16), (33, 9, 33), (64, 64, 64)])
def test_igemm_is_exact(m, k, n):
    s, av = _lcg(1, m * k, False)
    s, bv = _lcg(s, k * n, True)
    a = torch.tensor(av, dtype=torch.uint8)
    b = torch.tensor(bv, dtype=torch.int8)
    got = igemm(a, b, m, k, n)
    assert tuple(got.shape) == (m, n) and got.dtype == torch.int32
    assert torch.equal(got, igemm_scalar(a, b, m, k, n))
    i, j = m // 2, n // 2                                                       # one entry by hand
    assert int(got[i, j]) == sum(av[i * k + t] * bv[t * n + j] for t in range(k))
