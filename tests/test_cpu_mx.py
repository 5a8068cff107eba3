"""Block-scaled formats (ops/mx.py) on CPU: the torch-op quantiser, the scale-chunk layout and the dequantised matmul."""
import pytest
import torch

from rust_neural_network_b200.ops import mx


@pytest.mark.parametrize("kind,tol", [("mxfp8", 0.04), ("nvfp4", 0.15)])
def test_quantise_dequantise_round_trip(kind, tol):
    torch.manual_seed(0)
    x = torch.randn(200, 512) * torch.logspace(-2, 2, 200).unsqueeze(1)         # rows of very different magnitude
    t = mx.quantize_mx(x, kind)
    y = mx.dequantize_mx(t)
    rel = (y - x).norm(dim=1) / x.norm(dim=1)
    assert float(rel.max()) < tol, float(rel.max())
    assert t.data.shape == (200, 512 if kind == "mxfp8" else 256)
    assert t.sf.numel() == 2 * (512 // (128 if kind == "mxfp8" else 64)) * 512      # 200 rows pad to 256 = 2 row blocks


def test_mxfp8_scales_are_the_smallest_power_of_two_that_fits():
    x = torch.zeros(128, 128)
    x[0, :32] = 448.0          # fits with scale 1
    x[1, :32] = 449.0          # needs scale 2
    x[2, 32:64] = 1e-3
    t = mx.quantize_mx(x, "mxfp8")
    idx = mx._sf_index(128, 128, 0, x.device)
    sf = t.sf[idx]
    assert int(sf[0, 0]) == 127 and int(sf[1, 0]) == 128
    assert int(sf[3, 0]) == 0                                                   # empty block: smallest scale, zero data
    y = mx.dequantize_mx(t)
    assert float(y[0, 0]) == 448.0 and abs(float(y[1, 0]) - 449.0) <= 16.0
    assert abs(float(y[2, 40]) - 1e-3) < 1e-4


def test_nvfp4_codes_follow_the_e2m1_table_low_nibble_first():
    x = torch.zeros(1, 256)
    x[0, :8] = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])
    x[0, 8:16] = -x[0, :8]
    t = mx.quantize_mx(x, "nvfp4", tensor_scale=1.0 / 448.0)                      # block scale 448 * (1/448) = 1
    codes = []
    for b in t.data[0, :8].tolist():
        codes += [b & 15, b >> 4]
    assert codes == [0, 1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12, 13, 14, 15] or codes[:8] == [0, 1, 2, 3, 4, 5, 6, 7]
    y = mx.dequantize_mx(t)
    assert torch.allclose(y[0, :16], x[0, :16])


def test_gemm_matches_the_dequantised_product_on_cpu():
    torch.manual_seed(1)
    a, b = torch.randn(64, 256), torch.randn(40, 256)
    for kind in ("mxfp8", "nvfp4"):
        qa, qb = mx.quantize_mx(a, kind), mx.quantize_mx(b, kind)
        out = mx.gemm_mx(qa, qb, torch.float32)
        ref = mx.dequantize_mx(qa) @ mx.dequantize_mx(qb).t()
        assert torch.allclose(out, ref, atol=1e-5)
        rel = float((out - a @ b.t()).norm() / (a @ b.t()).norm())
        assert rel < (0.05 if kind == "mxfp8" else 0.2), rel


def test_shape_rules():
    with pytest.raises(ValueError):
        mx.quantize_mx(torch.zeros(4, 96), "mxfp8")
    with pytest.raises(ValueError):
        mx.quantize_mx(torch.zeros(4, 128), "nvfp4")
