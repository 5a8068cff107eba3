"""linear_attention.py, one test per behaviour of rust-nn src/linear_attention.rs:683-1010: the flat-buffer forward
against the O(N^2) double loop, the analytic gradients against central differences, and the autograd `Tensor` API."""
import math

import pytest
import torch

from rust_neural_network_b200.linear_attention import KernelKind, linear_attention_backward, linear_attention_forward
from rust_neural_network_b200.tensor import Tensor


def _lcg(seed, n):
    out = []
    for _ in range(n):
        seed = (seed * 1664525 + 1013904223) & 0xFFFFFFFF
        out.append((seed >> 8) / 16777216.0 - 0.5)
    return seed, out


def _phi(kind, x):
    return (x + 1.0 if x > 0 else math.exp(x)) if kind == KernelKind.Elu else max(x, 0.0) ** 2


def _naive(kind, q, k, v, seq, d, scale, eps, causal):
    out = [0.0] * (seq * d)
    for i in range(seq):
        acc, den = [0.0] * d, 0.0
        for j in range(seq):
            if causal and j > i:
                continue
            score = sum(_phi(kind, q[i * d + a] * scale) * _phi(kind, k[j * d + a] * scale) for a in range(d))
            for b in range(d):
                acc[b] += score * v[j * d + b]
            den += score
        for b in range(d):
            out[i * d + b] = acc[b] / (den + eps)
    return out


def _forward_case(seed, batch, seq, d, causal, kind):
    s, q = _lcg(seed, batch * seq * d)
    s, k = _lcg(s, batch * seq * d)
    s, v = _lcg(s, batch * seq * d)
    scale = 1.0 / math.sqrt(d)
    out = linear_attention_forward(q, k, v, batch, seq, d, scale, 1e-6, causal, kind).reshape(-1).tolist()
    sd = seq * d
    for b in range(batch):
        ref = _naive(kind, q[b * sd:], k[b * sd:], v[b * sd:], seq, d, scale, 1e-6, causal)
        assert max(abs(x - y) for x, y in zip(out[b * sd:(b + 1) * sd], ref)) < 1e-4


def test_forward_non_causal_elu_matches_the_double_loop():
    _forward_case(1, 2, 12, 8, False, KernelKind.Elu)


def test_forward_causal_elu_matches_the_double_loop():
    _forward_case(2, 2, 11, 7, True, KernelKind.Elu)


def test_forward_non_causal_relu2_matches_the_double_loop():
    _forward_case(3, 1, 14, 9, False, KernelKind.Relu2)


@pytest.mark.parametrize("causal,kind", [(False, KernelKind.Elu), (True, KernelKind.Elu), (False, KernelKind.Relu2)])
def test_gradients_match_central_differences(causal, kind):
    batch, seq, d = 1, 6, 4
    s, q = _lcg(11, seq * d)
    s, k = _lcg(s, seq * d)
    s, v = _lcg(s, seq * d)
    s, g = _lcg(s, seq * d)
    scale, eps = 1.0 / math.sqrt(d), 1e-6
    dq, dk, dv = (t.reshape(-1).tolist() for t in linear_attention_backward(q, k, v, g, batch, seq, d, scale, eps, causal, kind))

    def loss(q_, k_, v_):
        return sum(a * b for a, b in zip(_naive(kind, q_, k_, v_, seq, d, scale, eps, causal), g))

    h = 1e-3
    for which, analytic in enumerate((dq, dk, dv)):
        for i in range(0, seq * d, 5):
            args_hi, args_lo = [list(q), list(k), list(v)], [list(q), list(k), list(v)]
            args_hi[which][i] += h
            args_lo[which][i] -= h
            num = (loss(*args_hi) - loss(*args_lo)) / (2 * h)
            assert abs(num - analytic[i]) < 2e-3, (which, i, num, analytic[i])


def test_tensor_api_end_to_end_backward():
    batch, seq, d = 2, 16, 8
    q, k, v = (Tensor.randn([batch, seq, d]).set_requires_grad(True) for _ in range(3))
    out = Tensor.linear_attention(q, k, v, 1.0 / math.sqrt(d), 1e-6, False, KernelKind.Elu)
    assert list(out.shape()) == [batch, seq, d]
    out.sum().backward()
    for t in (q, k, v):
        assert list(t.grad().shape) == [batch, seq, d]
    q2, k2, v2 = (Tensor.randn([1, 12, 6]).set_requires_grad(True) for _ in range(3))      # the causal ReLU^2 path
    Tensor.linear_attention(q2, k2, v2, 0.5, 1e-6, True, KernelKind.Relu2).sum().backward()
    assert all(t.grad() is not None for t in (q2, k2, v2))
