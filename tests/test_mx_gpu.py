"""Block-scaled tensor-core GEMM (csrc/gemm/gemm_mx_sm100.cu): the CUDA quantiser against the torch-op quantiser, and the
`tcgen05.mma ... .block_scale` product against an fp32 matmul of the dequantised operands."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return float((a.float() - b.float()).norm() / (b.float().norm() + 1e-30))


@pytest.mark.parametrize("kind", ["mxfp8", "nvfp4"])
def test_cuda_quantiser_matches_torch_ops(kind):
    from rust_neural_network_b200.ops import mx
    torch.manual_seed(0)
    x = (torch.randn(300, 768) * torch.logspace(-2, 2, 300).unsqueeze(1)).cuda()
    ts = float(x.abs().max()) / (6 * 448)
    t = mx.quantize_mx(x, kind, tensor_scale=ts)
    data, sf = mx._quantize_torch(x, mx.KINDS[kind], ts if kind == "nvfp4" else 1.0)
    assert torch.equal(t.sf, sf)
    assert float((t.data != data).float().mean()) < 1e-3          # a tie at a rounding boundary may fall the other way
    d = mx.dequantize_mx(t)
    assert _rel(d, x) < (0.04 if kind == "mxfp8" else 0.15)
    tb = mx.quantize_mx(x.bfloat16(), kind, tensor_scale=ts)
    assert _rel(mx.dequantize_mx(tb), x) < (0.04 if kind == "mxfp8" else 0.15)


@pytest.mark.parametrize("kind", ["mxfp8", "nvfp4"])
@pytest.mark.parametrize("M,N,K", [(128, 256, 256), (200, 264, 512), (512, 1024, 2048), (1024, 384, 4096)])
def test_block_scaled_gemm_matches_dequantised_fp32_product(kind, M, N, K):
    from rust_neural_network_b200 import _native as nv
    from rust_neural_network_b200.ops import mx
    torch.manual_seed(M + N + K)
    # rows and K blocks of very different magnitude: a wrong scale factor (row, block or byte) cannot hide
    a = (torch.randn(M, K) * torch.logspace(-1, 1, M).unsqueeze(1) * (1 + torch.arange(K) // 64 % 5).float()).cuda()
    b = (torch.randn(N, K) * torch.logspace(1, -1, N).unsqueeze(1)).cuda()
    qa, qb = mx.quantize_mx(a, kind), mx.quantize_mx(b, kind)
    out = mx.gemm_mx(qa, qb, torch.float32)
    torch.cuda.synchronize(); nv.check_status()
    ref = mx.dequantize_mx(qa).double() @ mx.dequantize_mx(qb).double().t()
    assert _rel(out, ref) < 1e-5, _rel(out, ref)
    worst = float(((out.double() - ref).abs() / (ref.abs() + 1e-3 * ref.abs().max())).max())
    assert worst < 1e-3, worst
    out16 = mx.gemm_mx(qa, qb, torch.bfloat16)
    assert _rel(out16, ref) < 4e-3
    # against the unquantised product: the format's own error
    assert _rel(out, a.double() @ b.double().t()) < (0.05 if kind == "mxfp8" else 0.2)


def test_mx_linear_layer():
    from rust_neural_network_b200.ops import mx
    torch.manual_seed(3)
    w, bias = torch.randn(512, 1024).cuda() * 0.05, torch.randn(512).cuda()
    x = torch.randn(4, 60, 1024).cuda().bfloat16()
    ref = x.float() @ w.t() + bias
    for kind, tol in (("mxfp8", 0.05), ("nvfp4", 0.2)):
        lin = mx.MxLinear(w, bias, kind)
        y = lin(x)
        assert y.shape == (4, 60, 512) and y.dtype == torch.bfloat16
        assert _rel(y, ref) < tol
        assert lin.memory_bytes() < w.numel() * (1.1 if kind == "mxfp8" else 0.6) + 2048


def test_quantized_linear_nvfp4_tensor_core_path():
    from rust_neural_network_b200 import nn
    from rust_neural_network_b200.quantize import QuantFormat, QuantizedLinear
    torch.manual_seed(5)
    lin = nn.Linear(512, 256).to_device("cuda", torch.float32)
    x = torch.randn(40, 512, device="cuda")
    ref = x @ lin.weight.t() + lin.bias
    soft = QuantizedLinear.from_linear(lin, QuantFormat.NVFP4, 16)
    hard = QuantizedLinear.from_linear(lin, QuantFormat.NVFP4, 16, tensor_core=True)
    assert hard.mx is not None and soft.mx is None
    ys, yh = soft.forward(x), hard.forward(x)
    assert _rel(ys, ref) < 0.15 and _rel(yh, ref) < 0.2          # the second also quantises the activations to 4 bits
    with pytest.raises(ValueError):
        QuantizedLinear.from_linear(nn.Linear(100, 8).to_device("cuda", torch.float32), QuantFormat.NVFP4, 16, tensor_core=True)
