"""The C++ restatement of the reference's CPU kernels (csrc/cpu_ref) against PyTorch fp32: it is an oracle, so it is
pinned first. Shapes include odd sizes and the small-product path, like the reference's own blas tests
(rust-nn src/blas.rs:1196-1509)."""
import math

import pytest
import torch

from rust_neural_network_b200 import cpu_ref
from rust_neural_network_b200.ops.linear_attention import linear_attention_ref
from rust_neural_network_b200.ops.scan import selective_scan_ref
from rust_neural_network_b200.utils.lcg import lcg_tensor


@pytest.mark.parametrize("m,n,k", [(1, 1, 1), (3, 5, 7), (4, 16, 8), (33, 47, 129), (128, 256, 256), (130, 270, 300), (17, 1, 1000)])
@pytest.mark.parametrize("ta,tb", [(False, False), (False, True), (True, False), (True, True)])
def test_packed_sgemm_matches_torch(m, n, k, ta, tb):
    a = lcg_tensor((k, m) if ta else (m, k), seed=1)
    b = lcg_tensor((n, k) if tb else (k, n), seed=2)
    c = lcg_tensor((m, n), seed=3)
    got = cpu_ref.sgemm(a, b, ta, tb, alpha=0.5, beta=2.0, c=c, threads=2)
    want = 0.5 * ((a.t() if ta else a) @ (b.t() if tb else b)) + 2.0 * c
    assert torch.allclose(got, want, rtol=1e-4, atol=1e-3 * math.sqrt(k))


def test_sgemm_k_zero_scales_c():
    c = torch.ones(3, 4)
    got = cpu_ref.sgemm(torch.zeros(3, 0), torch.zeros(0, 4), beta=3.0, c=c)
    assert torch.equal(got, 3.0 * c)


@pytest.mark.parametrize("causal", [False, True])
def test_flash_attention_loop_matches_dense_softmax(causal):
    q, k, v = (lcg_tensor((2, 37, 16), seed=s) for s in (4, 5, 6))
    got = cpu_ref.flash_attention(q, k, v, causal=causal)
    s = q @ k.transpose(1, 2) / 4.0
    if causal:
        s = s.masked_fill(torch.ones(37, 37).triu(1).bool(), float("-inf"))
    assert torch.allclose(got, torch.softmax(s, -1) @ v, atol=1e-5)


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("kind", ["elu", "relu2"])
def test_linear_attention_recurrence_matches_quadratic_form(causal, kind):
    q, k, v = (lcg_tensor((2, 29, 8), seed=s) for s in (7, 8, 9))
    got = cpu_ref.linear_attention(q, k, v, scale=0.5, causal=causal, kind=kind)
    want = linear_attention_ref(q.unsqueeze(2), k.unsqueeze(2), v.unsqueeze(2), scale=0.5, causal=causal, kind=kind).squeeze(2)
    assert torch.allclose(got, want, atol=1e-4)


def test_selective_scan_layernorm_adam_fused_linear():
    u, dl = lcg_tensor((2, 19, 6), seed=1), lcg_tensor((2, 19, 6), seed=2).abs() * 0.1
    A, Bm, Cm = -lcg_tensor((6, 4), seed=3).abs(), lcg_tensor((2, 19, 4), seed=4), lcg_tensor((2, 19, 4), seed=5)
    assert torch.allclose(cpu_ref.selective_scan(u, dl, A, Bm, Cm), selective_scan_ref(u, dl, A, Bm, Cm), atol=1e-5)
    x, g, b = lcg_tensor((5, 12), seed=6), lcg_tensor((12,), seed=7), lcg_tensor((12,), seed=8)
    assert torch.allclose(cpu_ref.layer_norm(x, g, b), torch.nn.functional.layer_norm(x, (12,), g, b, 1e-5), atol=1e-5)
    p, gr = lcg_tensor((37,), seed=9).clone(), lcg_tensor((37,), seed=10)
    m, v = torch.zeros(37), torch.zeros(37)
    p0 = p.clone()
    cpu_ref.adam_update(p, gr, m, v, 0.9, 0.999, 1e-8, 0.01)
    m1, v1 = 0.1 * gr, 0.001 * gr * gr
    assert torch.allclose(p, p0 - 0.01 * m1 / (v1.sqrt() + 1e-8), atol=1e-6)
    w, bb = lcg_tensor((7, 12), seed=11), lcg_tensor((7,), seed=12)
    assert torch.allclose(cpu_ref.fused_linear(x, w, bb, "relu"), torch.relu(x @ w.t() + bb), atol=1e-5)


def test_cpu_mlp_step_matches_autograd_adam():
    """One native step (forward, CE, backward, Adam in the reference's form) against PyTorch autograd + the same update."""
    dims = [20, 16, 12, 5]
    net = cpu_ref.CpuMLP(dims, seed=3)
    Ws = [w.clone().requires_grad_(True) for w in net.W]
    bs = [b.clone().requires_grad_(True) for b in net.b]
    x = lcg_tensor((9, 20), seed=1)
    y = torch.tensor([0, 1, 2, 3, 4, 0, 1, 2, 3])
    h = x
    for i, (w, b) in enumerate(zip(Ws, bs)):
        h = h @ w.t() + b
        if i + 1 < len(Ws):
            h = torch.relu(h)
    loss = torch.nn.functional.cross_entropy(h, y)
    loss.backward()
    got = net.step(x, labels=y, lr=1e-2)
    assert got == pytest.approx(float(loss), rel=1e-5)
    lr_t = 1e-2 * math.sqrt(1 - 0.999) / (1 - 0.9)
    for w, wn in zip(Ws, net.W):
        m, v = 0.1 * w.grad, 0.001 * w.grad ** 2
        assert torch.allclose(wn, w.detach() - lr_t * m / (v.sqrt() + 1e-8), atol=1e-6)
    first = got
    for _ in range(30):
        last = net.step(x, labels=y, lr=1e-2)
    assert last < 0.5 * first
