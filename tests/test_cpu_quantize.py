"""quantize.py, one test per behaviour of rust-nn src/quantize.rs:727-900: the eight formats' round trips, compression
figures, the linear / model wrappers, and how the group size moves the error."""
import pytest
import torch

from rust_neural_network_b200 import nn
from rust_neural_network_b200.quantize import QuantFormat as F, QuantizedLinear, QuantizedModel, QuantizedTensor as QT


def test_int8_round_trip():
    t = torch.tensor([[0.1, 0.5, -0.3], [0.8, -0.9, 0.0]])
    d = QT.quantize(t, F.INT8, 0).dequantize()
    assert float((d - t).abs().max()) < 0.05
    assert float((d - t).abs().max()) <= 0.9 / 127 / 2 + 1e-6     # half a step of the one whole-tensor group


def test_int4_compression():
    q = QT.quantize(torch.randn(64, 128), F.INT4, 32)
    assert q.compression_ratio() > 5.0
    assert tuple(q.dequantize().shape) == (64, 128)


def test_nf4_error_against_int4_on_normal_data():
    torch.manual_seed(0)
    t = torch.randn(256)
    e_nf4 = QT.quantize(t, F.NF4, 64).quantization_error(t)
    e_int4 = QT.quantize(t, F.INT4, 64).quantization_error(t)
    assert e_nf4 <= e_int4 * 1.5


def test_nvfp4_round_trip_of_representable_values():
    t = torch.tensor([[0.0, 0.5], [1.0, -1.5], [3.0, -6.0], [2.0, -0.5]])
    d = QT.quantize(t, F.NVFP4, 8).dequantize().reshape(-1)
    assert abs(float(d[0])) < 0.01 and abs(float(d[5]) + 6.0) < 0.1
    assert torch.equal(d, t.reshape(-1))                           # scale max/6 = 1: every E2M1 magnitude is exact


def test_fp16_round_trip():
    t = torch.tensor([1.0, 0.5, -0.25, 100.0, -1000.0, 0.001])
    d = QT.quantize(t, F.FP16, 0).dequantize()
    assert float(((d - t).abs() / t.abs().clamp_min(1e-6)).max()) < 0.01


def test_bf16_round_trip():
    t = torch.tensor([1.0, -2.5, 100.0, -1000.0])
    d = QT.quantize(t, F.BF16, 0).dequantize()
    assert float((d - t).abs().max()) < 1.0
    assert torch.equal(d, t)                                       # all four fit in 8 mantissa bits


def test_gguf_q4_round_trip():
    torch.manual_seed(1)
    t = torch.randn(32)
    q = QT.quantize(t, F.GGUF_Q4, 32)
    assert tuple(q.dequantize().shape) == (32,)
    assert q.quantization_error(t) < 0.5


def test_gguf_q8_error_is_small():
    torch.manual_seed(2)
    t = torch.randn(64)
    assert QT.quantize(t, F.GGUF_Q8, 32).quantization_error(t) < 0.05


def test_quantized_linear_forward():
    torch.manual_seed(3)
    layer = nn.Linear(8, 4)
    ql = QuantizedLinear.from_linear(layer, F.INT8, 0)
    x = torch.randn(2, 8)
    y = ql.forward(x)
    assert tuple(y.shape) == (2, 4)
    want = x @ layer.weight.detach().t() + layer.bias.detach()
    assert float((y.float() - want).abs().max()) < 0.05


def test_quantized_model_compression():
    model = nn.Sequential().add(nn.Linear(64, 128)).add(nn.ReLU()).add(nn.Linear(128, 64))
    qm = QuantizedModel.from_model(model, F.INT4, 32)
    assert qm.compression_ratio() > 4.0
    assert len(qm.layers()) == 2


@pytest.mark.parametrize("fmt", [F.FP16, F.BF16, F.INT8, F.INT4, F.NF4, F.NVFP4, F.GGUF_Q4, F.GGUF_Q8])
def test_every_format_gives_finite_values_of_the_right_shape(fmt):
    torch.manual_seed(4)
    d = QT.quantize(torch.randn(16, 16), fmt, 32).dequantize()
    assert tuple(d.shape) == (16, 16) and bool(torch.isfinite(d).all())


def test_format_bits_and_compression():
    assert F.FP16.bits() == 16 and F.INT8.bits() == 8 and F.NF4.bits() == 4 and F.NVFP4.bits() == 4
    assert abs(F.INT4.compression_ratio() - 8.0) < 0.1


def test_fp16_special_values():
    t = torch.tensor([0.0, 1.0, float("inf"), -float("inf"), 1e6])
    d = QT.quantize(t, F.FP16, 0).dequantize()
    assert float(d[0]) == 0.0 and abs(float(d[1]) - 1.0) < 0.01
    assert float(d[2]) == float("inf") and float(d[3]) == -float("inf")
    assert float(d[4]) == float("inf")                             # beyond 65504: the exponent field saturates


def test_smaller_groups_have_lower_error():
    torch.manual_seed(5)
    t = torch.randn(256)
    assert QT.quantize(t, F.INT4, 32).quantization_error(t) <= QT.quantize(t, F.INT4, 256).quantization_error(t)
