"""Central finite differences against the analytic gradients of every differentiable op (the reference's
tests/grad_check.rs, tests/linear_fusion.rs:96, tests/flash_attention.rs, tests/selective_scan.rs and the inline checks of
src/linear_attention.rs:848-913, src/position.rs:572-620): h = 1e-3, tolerance 1e-3 + 1e-2 max(|analytic|, |numeric|),
loss = a fixed random weighting of the outputs so that no gradient direction cancels by symmetry."""
import math

import pytest
import torch

from rust_neural_network_b200 import loss as L
from rust_neural_network_b200.ops import functional as F
from rust_neural_network_b200.ops.linear_attention import linear_attention
from rust_neural_network_b200.ops.scan import causal_conv1d, selective_scan
from rust_neural_network_b200.position import RoPE
from rust_neural_network_b200.tensor import Tensor
from rust_neural_network_b200.utils.lcg import lcg_tensor

H = 1e-3


def check(fn, inputs, which=None, h=H):
    """fn(*tensors) -> scalar. Compares autograd with central differences for every element of the chosen inputs."""
    leaves = [t.clone().double().float().requires_grad_(True) for t in inputs]
    fn(*leaves).backward()
    for idx in (which if which is not None else range(len(inputs))):
        ana = leaves[idx].grad.reshape(-1)
        base = inputs[idx].clone()
        flat = base.reshape(-1)
        for e in range(flat.numel()):
            old = float(flat[e])
            flat[e] = old + h
            up = float(fn(*[base if j == idx else inputs[j] for j in range(len(inputs))]))
            flat[e] = old - h
            dn = float(fn(*[base if j == idx else inputs[j] for j in range(len(inputs))]))
            flat[e] = old
            num = (up - dn) / (2 * h)
            a = float(ana[e])
            assert abs(a - num) <= 1e-3 + 1e-2 * max(abs(a), abs(num)), (idx, e, a, num)


def wsum(out, seed=99):
    return (out.float() * lcg_tensor(tuple(out.shape), seed=seed)).sum()


def test_losses_match_numeric():
    p, t = lcg_tensor((3, 4), seed=1) * 0.8, lcg_tensor((3, 4), seed=2)
    check(lambda x: L.MSELoss()(x, t), [p])
    check(lambda x: L.MSELoss("mean")(x, t), [p])
    check(lambda x: L.L1Loss()(x, t + 0.05), [p])
    check(lambda x: L.HuberLoss(0.5)(x, t), [p])
    prob = torch.sigmoid(lcg_tensor((3, 4), seed=3))
    tgt = (lcg_tensor((3, 4), seed=4) > 0).float()
    check(lambda x: L.BCEWithLogitsLoss()(x, tgt), [p])
    check(lambda x: L.BCELoss()(x, tgt), [prob * 0.8 + 0.1])
    onehot = torch.nn.functional.one_hot(torch.tensor([0, 2, 3]), 4).float()
    check(lambda x: L.CrossEntropyLoss()(x, onehot), [p])
    check(lambda x: L.CrossEntropyLoss()(x, torch.tensor([0, 2, 3])), [p])


def test_matmul_and_broadcast_gradients_match_numeric():
    a, b = lcg_tensor((3, 4), seed=5), lcg_tensor((4, 2), seed=6)
    check(lambda x, y: wsum(Tensor(x).matmul(Tensor(y)).t), [a, b])
    bias = lcg_tensor((4,), seed=7)
    check(lambda x, y: wsum(Tensor(x).add(Tensor(y)).t), [a, bias])          # the bias gradient sums over the broadcast rows
    check(lambda x, y: wsum(Tensor(x).mul(Tensor(y)).t), [a, bias])
    check(lambda x, y: wsum(Tensor(x).sub(Tensor(y)).t), [a, bias])


@pytest.mark.parametrize("act", ["none", "relu", "gelu", "silu", "sigmoid", "tanh"])
def test_fused_linear_gradients_match_numeric(act):
    x, w, b = lcg_tensor((5, 6), seed=8) + 0.013, lcg_tensor((4, 6), seed=9), lcg_tensor((4,), seed=10)
    check(lambda xx, ww, bb: wsum(F.linear(xx, ww, bb, act, None)), [x, w, b])
    r = lcg_tensor((5, 4), seed=11)
    check(lambda xx, rr: wsum(F.linear(xx, w, b, act, rr)), [x, r])


def test_activations_layernorm_softplus_match_numeric():
    x = lcg_tensor((3, 8), seed=12) * 2 + 0.017
    for fn in (F.relu, F.sigmoid, F.tanh, F.gelu, F.silu, F.softplus):
        check(lambda t: wsum(fn(t)), [x])
    g, b = lcg_tensor((8,), seed=13) + 1.5, lcg_tensor((8,), seed=14)
    check(lambda t, gg, bb: wsum(F.layer_norm(t, gg, bb, 1e-5)), [x, g, b])
    check(lambda t: wsum(F.softmax(t)), [x])


@pytest.mark.parametrize("causal", [False, True])
def test_flash_attention_gradients_match_numeric(causal):
    q, k, v = (lcg_tensor((1, 6, 2, 4), seed=s) for s in (15, 16, 17))
    check(lambda a, b, c: wsum(F.flash_attention(a, b, c, scale=0.5, causal=causal)), [q, k, v])


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("kind", ["elu", "relu2"])
def test_linear_attention_gradients_match_numeric(causal, kind):
    q, k, v = (lcg_tensor((1, 7, 1, 3), seed=s) + 0.021 for s in (18, 19, 20))
    check(lambda a, b, c: wsum(linear_attention(a, b, c, scale=0.7, causal=causal, kind=kind, chunk=4)), [q, k, v])


def test_selective_scan_and_conv_gradients_match_numeric():
    u, dl = lcg_tensor((1, 5, 3), seed=21), lcg_tensor((1, 5, 3), seed=22).abs() * 0.3 + 0.05
    A, Bm, Cm = -lcg_tensor((3, 2), seed=23).abs() - 0.1, lcg_tensor((1, 5, 2), seed=24), lcg_tensor((1, 5, 2), seed=25)
    check(lambda a, b, c, d, e: wsum(selective_scan(a, b, c, d, e)), [u, dl, A, Bm, Cm])
    z, dsk, db = lcg_tensor((1, 5, 3), seed=26), lcg_tensor((3,), seed=27), lcg_tensor((3,), seed=28) * 0.1
    check(lambda a, b, zz, dd, bb: wsum(selective_scan(a, b, A, Bm, Cm, dd, zz, bb, True)), [u, dl, z, dsk, db])
    x, w, cb = lcg_tensor((2, 6, 3), seed=29), lcg_tensor((3, 4), seed=30), lcg_tensor((3,), seed=31)
    check(lambda a, b, c: wsum(causal_conv1d(a, b, c, "silu")), [x, w, cb])
    check(lambda a, b: wsum(causal_conv1d(a, b, None, "none")), [x, w])


def test_rope_gradient_matches_numeric_and_preserves_norm():
    rope = RoPE(8, 16)
    x = lcg_tensor((2, 5, 8), seed=32)
    check(lambda t: wsum(rope.apply(t)), [x])
    y = rope.apply(x)
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1), atol=1e-5)


def test_embedding_and_lm_head_ce_match_numeric():
    from rust_neural_network_b200.ops.transformer import lm_head_ce
    table = lcg_tensor((6, 4), seed=33)
    ids = torch.tensor([[0, 3, 5], [2, 2, 1]])
    check(lambda t: wsum(F.embedding(ids, t)), [table])
    h, w, b = lcg_tensor((2, 3, 4), seed=34), lcg_tensor((6, 4), seed=35), lcg_tensor((6,), seed=36)
    labels = torch.tensor([[1, 0, 5], [2, 3, 3]])
    check(lambda hh, ww, bb: lm_head_ce(hh, ww, bb, labels), [h, w, b])
