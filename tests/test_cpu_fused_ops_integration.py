"""The fused autograd ops through the reference-shaped `Tensor` API, one test per behaviour of rust-nn
tests/linear_fusion.rs:8-163, tests/selective_scan.rs:19-145 and tests/flash_attention.rs:45-157: values against plain
loops, gradients against central differences."""
import math

import torch

from rust_neural_network_b200 import nn
from rust_neural_network_b200.models.looped_transformer import AttentionKind, Transformer
from rust_neural_network_b200.optim import Adam
from rust_neural_network_b200.tensor import Tensor


def leaf(data, shape):
    return Tensor.new(torch.tensor(data, dtype=torch.float32).reshape(shape), True)


def _scalar(t):
    return float((t.t if isinstance(t, Tensor) else t).detach().reshape(-1)[0])


def _central(fn, base, shape, idxs=None, eps=1e-3):
    out = {}
    for i in (idxs if idxs is not None else range(len(base))):
        hi, lo = list(base), list(base)
        hi[i] += eps
        lo[i] -= eps
        out[i] = (_scalar(fn(leaf(hi, shape))) - _scalar(fn(leaf(lo, shape)))) / (2 * eps)
    return out


# ------------------------------------------------------------------ fused Linear
def test_fused_linear_forward_matches_the_triple_loop():
    torch.manual_seed(0)
    lin = nn.Linear(5, 3)
    x = torch.randn(4, 5)
    y = lin(x).detach()
    assert list(y.shape) == [4, 3]
    w, b = lin.weight.detach(), lin.bias.detach()
    for i in range(4):
        for o in range(3):
            s = sum(float(x[i, p]) * float(w[o, p]) for p in range(5)) + float(b[o])
            assert abs(float(y[i, o]) - s) < 1e-4


def test_linear_backward_matches_central_differences_on_every_weight():
    torch.manual_seed(1)
    lin = nn.Linear(4, 3)
    x, target = torch.randn(3, 4), torch.randn(3, 3)
    ((lin(x) - target) ** 2).sum().backward()
    g = lin.weight.grad.reshape(-1).tolist()
    assert any(abs(v) > 1e-4 for v in g)
    flat = lin.weight.data.view(-1)
    h = 1e-3
    sse = lambda: float(((lin(x).detach() - target) ** 2).sum())
    for i in range(flat.numel()):
        keep = float(flat[i])
        flat[i] = keep + h
        lp = sse()
        flat[i] = keep - h
        lm = sse()
        flat[i] = keep
        num = (lp - lm) / (2 * h)
        assert abs(num - g[i]) < 1e-3 + 1e-2 * max(abs(num), abs(g[i])), (i, num, g[i])


def test_small_mlp_learns():
    torch.manual_seed(2)
    model = (nn.Sequential().add(nn.Linear(6, 16)).add(nn.ReLU()).add(nn.Linear(16, 8)).add(nn.ReLU()).add(nn.Linear(8, 1)))
    opt = Adam(model.parameters(), lr=0.05)
    x, target = torch.randn(16, 6), torch.randn(16, 1)
    mse = lambda: float(((model(x).detach() - target) ** 2).mean())
    loss0 = mse()
    for _ in range(40):
        opt.zero_grad()
        ((model(x) - target) ** 2).sum().backward()
        opt.step()
    assert mse() < 0.5 * loss0


def test_transformer_with_linear_attention_runs_and_is_differentiable():
    model = Transformer(8, 16, 2, 32, 8, 2).with_attention(AttentionKind.Linear)
    y = model(torch.randn(2, 6, 8))
    assert list(y.shape) == [2, 6, 8]
    y.sum().backward()
    assert sum(p.grad is not None for p in model.parameters()) > 0


def test_transformer_with_flash_attention_runs():
    model = Transformer(8, 16, 2, 32, 8, 2)
    y = model(torch.randn(2, 6, 8))
    assert list(y.shape) == [2, 6, 8]
    y.sum().backward()
    assert all(p.grad is not None for p in model.parameters())


# ------------------------------------------------------------------ selective scan
def _scan_inputs(batch, seq, dim, n):
    delta = leaf([0.2 + 0.01 * i for i in range(batch * seq * dim)], [batch, seq, dim])
    bv = leaf([0.4 - 0.02 * i for i in range(batch * seq * n)], [batch, seq, n])
    cv = leaf([0.3 + 0.03 * i for i in range(batch * seq * n)], [batch, seq, n])
    u = leaf([0.6 - 0.05 * i for i in range(batch * seq * dim)], [batch, seq, dim])
    a = leaf([-0.5 - 0.1 * i for i in range(dim * n)], [dim, n])
    return delta, bv, cv, u, a


def test_selective_scan_forward_shape_and_recurrence():
    batch, seq, dim, n = 2, 5, 4, 3
    delta, bv, cv, u, a = _scan_inputs(batch, seq, dim, n)
    y = Tensor.selective_scan(delta, bv, cv, u, a)
    assert list(y.shape()) == [batch, seq, dim]
    d_, b_, c_, u_, a_ = (t.t.detach() for t in (delta, bv, cv, u, a))       # h_t = exp(delta A) h_{t-1} + delta B u; y = C . h
    h = torch.zeros(batch, dim, n)
    for t in range(seq):
        h = torch.exp(d_[:, t, :, None] * a_) * h + d_[:, t, :, None] * b_[:, t, None, :] * u_[:, t, :, None]
        assert torch.allclose(y.t.detach()[:, t], (h * c_[:, t, None, :]).sum(-1), atol=1e-5)


def _scan_grad_case(which):
    batch, seq, dim, n = 1, 4, 3, 2
    ts = list(_scan_inputs(batch, seq, dim, n))
    Tensor.selective_scan(*ts).sum().backward()
    analytic = ts[which].grad().reshape(-1).tolist()
    base, shape = ts[which].t.detach().reshape(-1).tolist(), list(ts[which].t.shape)

    def fn(t):
        args = list(ts)
        args[which] = t
        return Tensor.selective_scan(*args).sum()

    num = _central(fn, base, shape)
    assert max(abs(num[i] - analytic[i]) for i in num) < 1e-2


def test_selective_scan_grad_a_matches_numeric():
    _scan_grad_case(4)


def test_selective_scan_grad_delta_matches_numeric():
    _scan_grad_case(0)


def test_selective_scan_grads_b_c_u_match_numeric():
    for which in (1, 2, 3):
        _scan_grad_case(which)


# ------------------------------------------------------------------ flash attention
def _flash_inputs():
    b, n, d = 2, 5, 4
    q = [math.sin(i * 0.13 - 1.0) for i in range(b * n * d)]
    k = [math.cos(i * 0.27 + 0.5) for i in range(b * n * d)]
    v = [math.tan(i * 0.09) * 0.1 for i in range(b * n * d)]
    return (b, n, d), q, k, v


def test_flash_forward_matches_the_full_softmax():
    (b, n, d), q, k, v = _flash_inputs()
    scale = 1.0 / math.sqrt(d)
    out = Tensor.flash_attention(leaf(q, [b, n, d]), leaf(k, [b, n, d]), leaf(v, [b, n, d]), scale).t.detach()
    qt, kt, vt = (torch.tensor(t).reshape(b, n, d) for t in (q, k, v))
    ref = torch.softmax(qt @ kt.transpose(1, 2) * scale, -1) @ vt
    assert float((out - ref).abs().max()) < 1e-5


def _flash_grad_case(which):
    (b, n, d), q, k, v = _flash_inputs()
    scale = 1.0 / math.sqrt(d)
    ts = [leaf(q, [b, n, d]), leaf(k, [b, n, d]), leaf(v, [b, n, d])]
    w = Tensor.new(torch.linspace(-1.0, 1.0, b * n * d).reshape(b, n, d))     # weighted sum: the plain sum has a zero q-gradient
    Tensor.flash_attention(*ts, scale).mul(w).sum().backward()
    analytic = ts[which].grad().reshape(-1).tolist()

    def fn(t):
        args = list(ts)
        args[which] = t
        return Tensor.flash_attention(*args, scale).mul(w).sum()

    num = _central(fn, (q, k, v)[which], [b, n, d], idxs=range(0, b * n * d, 3))
    assert max(abs(num[i] - analytic[i]) for i in num) < 2e-3


def test_flash_grad_q_matches_numeric():
    _flash_grad_case(0)


def test_flash_grad_k_and_v_match_numeric():
    _flash_grad_case(1)
    _flash_grad_case(2)
