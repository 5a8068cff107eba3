"""Position encodings, one test per property the reference checks (rust-nn src/position.rs:508-784): RoPE shape / norm /
identity at position 0 / relative-position property / YaRN / extend, CARoPE, ALiBi, sinusoidal and learned encodings,
the `PositionalEncoding` switch."""
import math

import pytest
import torch

from rust_neural_network_b200.position import (AlibiBias, CARoPE, LearnedPE, PositionalEncoding, RoPE, SinusoidalPE, alibi_slopes,
                                               inv_freq, inv_freq_yarn)
from rust_neural_network_b200.utils.lcg import lcg_tensor


def test_rope_preserves_shape():
    r = RoPE.new(8, 32)
    for shape in ((5, 8), (2, 5, 8), (2, 3, 5, 8)):
        assert r.apply(lcg_tensor(shape, seed=1)).shape == shape


def test_rope_preserves_norm():
    x = lcg_tensor((3, 16, 8), seed=2)
    assert torch.allclose(RoPE.new(8, 16).apply(x).norm(dim=-1), x.norm(dim=-1), atol=1e-5)


def test_rope_position_zero_is_identity():
    x = lcg_tensor((4, 8), seed=3)
    assert torch.allclose(RoPE.new(8, 4).apply(x)[0], x[0], atol=1e-6)
    assert not torch.allclose(RoPE.new(8, 4).apply(x)[3], x[3], atol=1e-3)


def test_rope_scores_depend_on_relative_position_only():
    """<R_m q, R_n k> is a function of m - n: shifting both positions leaves every score unchanged."""
    r = RoPE.new(16, 64)
    q, k = lcg_tensor((16,), seed=4), lcg_tensor((16,), seed=5)
    seq_q, seq_k = q.repeat(64, 1), k.repeat(64, 1)
    rq, rk = r.apply(seq_q), r.apply(seq_k)
    s = rq @ rk.t()
    for off in (1, 5, 17):
        d = torch.diagonal(s, offset=off)
        assert torch.allclose(d, d[0].expand_as(d), atol=1e-4)


def test_rope_differentiable():
    x = lcg_tensor((2, 6, 8), seed=6).requires_grad_(True)
    RoPE.new(8, 6).apply(x).pow(2).sum().backward()
    assert x.grad is not None and torch.isfinite(x.grad).all()
    assert torch.allclose(x.grad, 2 * x.detach(), atol=1e-5)         # a rotation: d|Rx|^2/dx = 2x


def test_rope_rejects_wrong_dim_and_long_sequences():
    r = RoPE.new(8, 4)
    with pytest.raises(ValueError):
        r.apply(torch.zeros(4, 6))
    with pytest.raises(ValueError):
        r.apply(torch.zeros(5, 8))


def test_rope_yarn_extends_context():
    base = inv_freq(16, 10000.0)
    yarn = inv_freq_yarn(16, 10000.0, 4.0)
    assert (yarn <= base + 1e-9).all() and yarn[-1] < base[-1]     # lower frequencies: longer wavelengths
    assert RoPE.yarn(16, 128, 10000.0, 4.0).apply(torch.ones(128, 16)).shape == (128, 16)
    assert RoPE.with_base(16, 8, 500.0).base == 500.0


def test_rope_extend_grows_tables():
    r = RoPE.new(8, 4)
    first = r.cos.clone()
    r.extend(16)
    assert r.max_seq_len == 16 and r.cos.shape[0] == 16 and torch.equal(r.cos[:4], first)
    r.extend(8)                                                     # never shrinks
    assert r.max_seq_len == 16


def test_carope_preserves_shape():
    c = CARoPE(8, 12, 16)
    assert c.apply(lcg_tensor((2, 10, 8), seed=7), lcg_tensor((10, 12), seed=8)).shape == (2, 10, 8)


def test_carope_different_from_static_rope():
    torch.manual_seed(0)
    c = CARoPE(8, 12, 16).with_spread(0.5)
    x, emb = lcg_tensor((10, 8), seed=9), lcg_tensor((10, 12), seed=10) * 5
    out = c.apply(x, emb)
    assert not torch.allclose(out, RoPE.new(8, 16).apply(x), atol=1e-4)
    assert torch.allclose(out.norm(dim=-1), x.norm(dim=-1), atol=1e-5)          # still a rotation
    zero = CARoPE(8, 12, 16).with_spread(0.0)
    assert torch.allclose(zero.apply(x, emb), RoPE.new(8, 16).apply(x), atol=1e-5)


def test_carope_has_parameters():
    ps = CARoPE(8, 12, 16).parameters()
    assert len(ps) == 1 and tuple(ps[0].shape) == (12, 4) and ps[0].requires_grad


def test_alibi_diagonal_is_zero():
    b = AlibiBias(4).bias_matrix(6)
    assert b.shape == (4, 6, 6) and float(torch.diagonal(b, dim1=1, dim2=2).abs().max()) == 0.0


def test_alibi_farther_is_more_negative():
    b = AlibiBias(2).bias_matrix(8)
    assert (b <= 0).all() and b[0, 7, 0] < b[0, 7, 6] < 0 and torch.allclose(b, b.transpose(1, 2))


def test_alibi_slopes_decreasing():
    s = alibi_slopes(8)
    assert all(a > b for a, b in zip(s, s[1:])) and s[0] == pytest.approx(0.5) and s[-1] == pytest.approx(2.0 ** -8)
    a = AlibiBias(8)
    assert a.slope(0) == s[0] and a.slope(99) == 0.0


def test_sinusoidal_pe_correct_values():
    t = SinusoidalPE(6, 10).table()
    assert t.shape == (10, 6) and torch.allclose(t[0], torch.tensor([0.0, 1.0, 0.0, 1.0, 0.0, 1.0]))
    assert t[3, 0] == pytest.approx(math.sin(3.0)) and t[3, 1] == pytest.approx(math.cos(3.0))
    assert t[3, 2] == pytest.approx(math.sin(3.0 / 10000 ** (2 / 6)), rel=1e-5)
    x = torch.zeros(2, 4, 6)
    assert torch.allclose(SinusoidalPE(6, 10).apply(x)[1], t[:4])
    with pytest.raises(ValueError):
        SinusoidalPE(6, 3).apply(x)


def test_learned_pe_is_trainable():
    pe = LearnedPE(4, 8)
    x = torch.zeros(2, 5, 4)
    pe.apply(x).sum().backward()
    g = pe.parameters()[0].grad
    assert torch.equal(g[:5], torch.full((5, 4), 2.0)) and float(g[5:].abs().sum()) == 0.0


def test_learned_pe_init_sinusoidal():
    pe = LearnedPE(6, 10).init_sinusoidal()
    assert torch.allclose(pe.parameters()[0].detach(), SinusoidalPE(6, 10).table())


def test_positional_encoding_enum():
    x = torch.ones(1, 3, 4)
    assert torch.equal(PositionalEncoding.none().apply(x), x) and PositionalEncoding.none().parameters() == []
    s = PositionalEncoding.sinusoidal(4, 8)
    assert not torch.equal(s.apply(x), x) and s.parameters() == []
    l = PositionalEncoding.learned(4, 8)
    assert len(l.parameters()) == 1 and l.apply(x).shape == x.shape
