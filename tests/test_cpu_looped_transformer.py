"""The looped transformer, multi-head attention, LayerNorm and permute, one test per behaviour of rust-nn
tests/looped_transformer.rs:18-317, through the reference-shaped `Tensor` API."""
import math

import torch

from rust_neural_network_b200 import nn
from rust_neural_network_b200.models.looped_transformer import LoopedTransformer, MultiHeadAttention, Transformer
from rust_neural_network_b200.optim import Adam
from rust_neural_network_b200.tensor import Tensor


def leaf(data, shape):
    return Tensor.new(torch.tensor(data, dtype=torch.float32).reshape(shape), True)


def _raw(y):
    return y.t if isinstance(y, Tensor) else y


def _numeric(fn, base, shape, eps=1e-3):
    out = []
    for i in range(len(base)):
        hi, lo = list(base), list(base)
        hi[i] += eps
        lo[i] -= eps
        out.append((float(_raw(fn(leaf(hi, shape)).sum()).detach()) - float(_raw(fn(leaf(lo, shape)).sum()).detach())) / (2 * eps))
    return out


# ------------------------------------------------------------------ permute
def test_permute_swaps_axes():
    p = leaf([1.0, 2.0, 3.0, 4.0, 5.0, 6.0], [2, 3]).permute([1, 0])
    assert list(p.shape()) == [3, 2]
    assert (p.get([0, 0]), p.get([0, 1]), p.get([1, 0]), p.get([2, 0])) == (1.0, 4.0, 2.0, 3.0)


def test_permute_4d_head_rearrange():
    assert list(Tensor.randn([2, 3, 2, 4]).permute([0, 2, 1, 3]).shape()) == [2, 2, 3, 4]


def test_permute_backward_matches_numeric():
    base, shape = [0.3, -0.1, 0.5, 0.2, -0.4, 0.6], [2, 3]
    w = torch.arange(1.0, 7.0).reshape(3, 2)                       # a weighted sum, so that a wrong axis order shows
    fn = lambda t: t.permute([1, 0]).mul(Tensor.new(w))
    t = leaf(base, shape)
    fn(t).sum().backward()
    num = _numeric(fn, base, shape)
    assert max(abs(a - b) for a, b in zip(t.grad().reshape(-1).tolist(), num)) < 2e-3
    assert torch.equal(t.grad(), w.t())


# ------------------------------------------------------------------ LayerNorm
def test_layernorm_normalizes_last_axis():
    y = _raw(nn.LayerNorm(4)(leaf([1.0, 2.0, 3.0, 4.0, 5.0, 6.0, 7.0, 8.0], [2, 4]))).detach()
    assert float(y.mean(-1).abs().max()) < 1e-4
    assert torch.allclose(y.var(-1, unbiased=False), torch.ones(2), atol=1e-3)


def test_layernorm_grad_matches_numeric():
    base, shape = [0.3, -0.1, 0.5, 0.2, -0.4, 0.6], [2, 3]
    gamma, beta = leaf([1.0, 1.5, 0.5], [3]), leaf([0.0, 0.0, 0.0], [3])
    fn = lambda t: t.layer_norm(gamma, beta, 1e-5)
    x = leaf(base, shape)
    fn(x).sum().backward()
    num = _numeric(fn, base, shape)
    assert max(abs(a - b) for a, b in zip(x.grad().reshape(-1).tolist(), num)) < 1e-2


def test_layernorm_gamma_grad_nonzero():
    ln = nn.LayerNorm(4)
    _raw(ln(Tensor.randn([2, 3, 4]))).sum().backward()
    assert ln.gamma.grad is not None and bool((ln.gamma.grad.abs() > 1e-6).any())


# ------------------------------------------------------------------ multi-head attention
def test_mha_preserves_shape():
    assert list(_raw(MultiHeadAttention(16, 4)(torch.randn(2, 5, 16))).shape) == [2, 5, 16]


def test_mha_single_head_is_scaled_dot_product_attention():
    torch.manual_seed(0)
    mha = MultiHeadAttention(8, 1)
    x = torch.randn(1, 4, 8)
    y = _raw(mha(x)).detach()
    assert list(y.shape) == [1, 4, 8] and bool(torch.isfinite(y).all())
    ps = [p.detach() for p in mha.parameters()]                     # wq bq wk bk wv bv wo bo
    q, k, v = (x @ ps[i].t() + ps[i + 1] for i in (0, 2, 4))
    want = torch.softmax(q @ k.transpose(1, 2) / math.sqrt(8), -1) @ v @ ps[6].t() + ps[7]
    assert torch.allclose(y, want, atol=1e-4)


def test_mha_is_differentiable():
    x = torch.tensor([math.sin(i * 0.01) for i in range(48)]).reshape(2, 3, 8).requires_grad_(True)
    _raw(MultiHeadAttention(8, 2)(x)).sum().backward()
    assert x.grad is not None and bool((x.grad.abs() > 0).any())


# ------------------------------------------------------------------ looped transformer
def test_looped_transformer_preserves_shape():
    model = LoopedTransformer(8, 16, 4, 32, 5, 4)
    assert list(model(torch.randn(2, 6, 8)).shape) == [2, 6, 5]
    y = model.forward(Tensor.randn([2, 6, 8]))                      # the reference-shaped call: wrapper in, wrapper out
    assert isinstance(y, Tensor) and list(y.shape()) == [2, 6, 5]


def test_looped_transformer_is_differentiable_through_every_loop():
    model = LoopedTransformer(6, 8, 2, 16, 3, 2)
    x = torch.tensor([math.sin(i * 0.05) for i in range(18)]).reshape(1, 3, 6).requires_grad_(True)
    _raw(model(x)).sum().backward()
    assert bool((x.grad.abs() > 0).any())
    assert all(p.grad is not None for p in model.parameters())


def test_adaptive_halting_stops_within_the_loop_budget():
    model = LoopedTransformer(4, 8, 2, 16, 2, 10).with_adaptive_halting(0.0)
    y, loops = model.forward_with_loops(torch.randn(1, 3, 4))
    assert list(_raw(y).shape) == [1, 3, 2]
    assert loops == 1                                               # threshold 0: the first sigmoid already reaches it


def test_looped_has_fewer_parameters_than_standard():
    looped, standard = LoopedTransformer(16, 32, 4, 64, 16, 8), Transformer(16, 32, 4, 64, 16, 8)
    assert len(looped.parameters()) < len(standard.parameters())
    assert sum(p.numel() for p in looped.parameters()) < sum(p.numel() for p in standard.parameters())


def test_looped_transformer_learns_the_copy_task():
    torch.manual_seed(0)
    model = LoopedTransformer(4, 12, 3, 24, 4, 3)
    opt = Adam(model.parameters(), lr=0.01)
    x = torch.tensor([0.3, -0.1, 0.5, 0.2, -0.4, 0.6, 0.1, -0.3, 0.2, 0.4, -0.5, 0.0]).reshape(1, 3, 4)
    losses = []
    for _ in range(60):
        opt.zero_grad()
        loss = ((_raw(model(x)) - x) ** 2).sum()
        loss.backward()
        opt.step()
        losses.append(float(loss))
    assert losses[-1] < 0.5 * losses[0]


def test_standard_transformer_preserves_shape():
    assert list(_raw(Transformer(8, 16, 4, 32, 5, 3)(torch.randn(2, 6, 8))).shape) == [2, 6, 5]


def test_more_loops_keep_shape_and_stay_finite():
    x = torch.randn(1, 3, 4)
    for loops in (4, 8):
        y = _raw(LoopedTransformer(4, 8, 2, 16, 4, loops)(x)).detach()
        assert list(y.shape) == [1, 3, 4] and bool(torch.isfinite(y).all())
