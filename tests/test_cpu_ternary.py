"""ternary.py, one test per behaviour of rust-nn src/ternary.rs:370-515: {-1, 0, +1} quantisation with a per-row scale,
16 codes per 32-bit word, the layer and model wrappers and their compression / sparsity figures."""
import torch

from rust_neural_network_b200 import nn
from rust_neural_network_b200 import ternary as T


def test_quantize_produces_three_levels_per_row():
    t = torch.tensor([[0.5, -0.3, 0.01, -0.8], [0.6, -0.02, 0.9, -0.4]])
    q = T.TernaryTensor.quantize(t)
    d = q.dequantize()
    assert tuple(d.shape) == (2, 4) and float(d.abs().max()) < 2.0
    for r in range(2):                                            # every row: values in {-s, 0, +s} with s = mean |w| of the row
        s = float(t[r].abs().mean())
        assert all(min(abs(float(v) - c) for c in (-s, 0.0, s)) < 1e-5 for v in d[r])
    assert float(d[0, 2]) == 0.0 and float(d[1, 1]) == 0.0        # below 0.7 * mean |w|: zero


def test_compression_ratio():
    q = T.TernaryTensor.quantize(torch.randn(64, 128))
    assert q.mem_bytes() == 64 * 128 // 16 * 4 + 64 * 4           # 2 bits per weight + one fp32 scale per row
    assert q.compression_ratio() > 10.0


def test_sparsity_is_nonzero():
    q = T.TernaryTensor.quantize(torch.tensor([[0.5, -0.5, 0.01, -0.01], [0.5, -0.5, 0.01, -0.01]]))
    assert q.sparsity() == 0.5


def test_value_counts():
    q = T.TernaryTensor.quantize(torch.tensor([[10.0, -10.0, 0.001, -0.001], [10.0, -10.0, 10.0, -10.0]]))
    pos, neg, zero = q.value_counts()
    assert pos + neg + zero == 8 and (pos, neg, zero) == (3, 3, 2)


def test_pack_unpack_round_trip():
    values = [1, -1, 0, 1, -1, 0, 1, 1, -1, -1, 0, 0, 1, -1, 1, 0]
    packed = T.pack_ternary(values)
    assert len(packed) == 1
    assert T.unpack_ternary(packed, 16) == values


def test_pack_unpack_large_with_a_ragged_tail():
    values = [(1, -1, 0)[i % 3] for i in range(1000)]
    packed = T.pack_ternary(values)
    assert len(packed) == 63                                      # ceil(1000 / 16)
    assert T.unpack_ternary(packed, 1000) == values


def test_linear_forward_shape_and_values():
    torch.manual_seed(0)
    layer = nn.Linear(8, 4)
    tl = T.TernaryLinear.from_linear(layer)
    x = torch.randn(2, 8)
    y = tl.forward(x)
    assert tuple(y.shape) == (2, 4) and bool(torch.isfinite(y).all())
    want = x @ tl.ternary_weight.dequantize().reshape(4, 8).t() + layer.bias.detach()
    assert torch.allclose(y.float(), want, atol=1e-4)


def test_linear_is_sums_and_differences_of_inputs():
    layer = nn.Linear(4, 2)
    tl = T.TernaryLinear.from_linear(layer)
    x = torch.tensor([[1.0, 2.0, 3.0, 4.0]])
    y = tl.forward(x)
    assert tuple(y.shape) == (1, 2)
    codes = tl.ternary_weight.values().reshape(2, 4)                                    # {-1, 0, +1}
    assert set(codes.reshape(-1).tolist()) <= {-1.0, 0.0, 1.0}
    want = (codes @ x[0]) * tl.ternary_weight.scales + layer.bias.detach()
    assert torch.allclose(y[0].float(), want, atol=1e-5)


def test_model_compression():
    model = nn.Sequential().add(nn.Linear(32, 64)).add(nn.ReLU()).add(nn.Linear(64, 32))
    assert T.TernaryModel.from_model(model).compression_ratio() > 8.0


def test_model_forward():
    model = nn.Sequential().add(nn.Linear(8, 16)).add(nn.ReLU()).add(nn.Linear(16, 4))
    tm = T.TernaryModel.from_model(model)
    x = torch.randn(2, 8)
    assert tuple(tm.forward_first_layer(x).shape) == (2, 16)
    assert tuple(tm.forward(x).shape) == (2, 4)


def test_model_sparsity_is_a_fraction():
    tm = T.TernaryModel.from_model(nn.Sequential().add(nn.Linear(16, 32)))
    assert 0.0 <= tm.avg_sparsity() <= 1.0


def test_quantization_error_is_below_the_spread_of_the_data():
    torch.manual_seed(2)
    t = torch.randn(64)
    q = T.ternarize(t)
    assert q.quantization_error(t) < 1.5
