"""GPU tests: the 8-bit tensor-core GEMM kinds and the quantisation kernels against their fp32 /
integer PyTorch restatements."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from rust_neural_network_b200 import nn, int8, quantize as qz, quant, ternary, compression as cp
from rust_neural_network_b200.ops import gemm as G
from rust_neural_network_b200.ops import quant_kernels as Q

DEV = "cuda"


def _rand_i8(shape, g, lo=-128, hi=128):
    return torch.randint(lo, hi, shape, generator=g, dtype=torch.int32).to(torch.int8)


@pytest.mark.parametrize("M,N,K", [(128, 128, 128), (300, 200, 416), (1024, 768, 2048), (64, 256, 4096)])
@pytest.mark.parametrize("unsigned_a", [False, True])
def test_int8_gemm_exact(M, N, K, unsigned_a):
    g = torch.Generator().manual_seed(M + N + K)
    a = (torch.randint(0, 256, (M, K), generator=g, dtype=torch.int32).to(torch.uint8) if unsigned_a else _rand_i8((M, K), g)).to(DEV)
    b = _rand_i8((N, K), g).to(DEV)
    out = G.gemm(a, b, out_dtype=torch.int32)
    want = (a.cpu().to(torch.int64) @ b.cpu().to(torch.int64).t()).to(torch.int32)
    assert out.dtype == torch.int32 and torch.equal(out.cpu(), want)


@pytest.mark.parametrize("bn", [128, 256])
@pytest.mark.parametrize("act", ["none", "gelu"])
def test_int8_gemm_scaled_epilogue(bn, act):
    g = torch.Generator().manual_seed(3)
    M, N, K = 520, 384, 640
    a, b = _rand_i8((M, K), g).to(DEV), _rand_i8((N, K), g).to(DEV)
    rs = (torch.rand(M, generator=g) * 0.01 + 0.001).to(DEV)
    cs = (torch.rand(N, generator=g) * 0.01 + 0.001).to(DEV)
    bias = torch.randn(N, generator=g).to(DEV)
    want = G.gemm_ref(a.cpu(), b.cpu(), row_scale=rs.cpu(), col_scale=cs.cpu(), bias=bias.cpu(), act=act, out_dtype=torch.float32)
    got = G.gemm(a, b, row_scale=rs, col_scale=cs, bias=bias, act=act, out_dtype=torch.float32, bn=bn)
    assert torch.allclose(got.cpu(), want, rtol=2e-3, atol=2e-3)
    got16 = G.gemm(a, b, row_scale=rs, col_scale=cs, bias=bias, act=act, bn=bn)
    assert got16.dtype == torch.bfloat16 and torch.allclose(got16.float().cpu(), want, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("M,N,K", [(256, 256, 256), (200, 136, 1000 + 24)])
def test_fp8_gemm(M, N, K):
    g = torch.Generator().manual_seed(5)
    a = (torch.randn(M, K, generator=g)).to(torch.float8_e4m3fn).to(DEV)
    b = (torch.randn(N, K, generator=g)).to(torch.float8_e4m3fn).to(DEV)
    cs = (torch.rand(N, generator=g) + 0.5).to(DEV)
    want = (a.cpu().float().double() @ b.cpu().float().double().t()).float() * cs.cpu()
    got = G.gemm(a, b, col_scale=cs, out_dtype=torch.float32)
    assert torch.allclose(got.cpu(), want, rtol=1e-3, atol=1e-2)


def test_quant_rows_matches_restatement():
    torch.manual_seed(0)
    for dt in (torch.float32, torch.bfloat16):
        x = (torch.randn(300, 1000) * 3).to(dt)
        x[7] = 0
        q_ref, s_ref = Q.quant_rows(x, "int8")
        q, s = Q.quant_rows(x.to(DEV), "int8")
        assert torch.allclose(s.cpu(), s_ref, rtol=1e-6)
        assert int((q.cpu().int() - q_ref.int()).abs().max()) <= 1          # a tie in x/scale may round either way after the division
        assert float((q.cpu().int() != q_ref.int()).float().mean()) < 1e-3
        q8, s8 = Q.quant_rows(x.to(DEV), "e4m3")
        back = q8.float().cpu() * s8.cpu()[:, None]
        assert float((back - x.float()).abs().max()) <= float(x.float().abs().max()) * 0.07


@pytest.mark.parametrize("fmt", [Q.Q_INT8, Q.Q_INT4, Q.Q_NF4, Q.Q_NVFP4, Q.Q_Q4_0, Q.Q_Q8_0])
@pytest.mark.parametrize("n,gs", [(4096, 64), (1000, 32), (777, 7), (5000, 5000)])
def test_group_quant_matches_restatement(fmt, n, gs):
    torch.manual_seed(n + gs + fmt)
    x = torch.randn(n)
    d_ref, s_ref = Q.quant_group(x, gs, fmt)
    d, s = Q.quant_group(x.to(DEV), gs, fmt)
    assert d.numel() == d_ref.numel() and torch.allclose(s.cpu(), s_ref, rtol=1e-6)
    mism = float((d.cpu() != d_ref).float().mean())
    assert mism < 2e-3                                                       # only exact rounding ties may differ
    deq_ref = Q.dequant_group(d.cpu(), s.cpu(), n, gs, fmt)
    for odt in (torch.float32, torch.bfloat16):
        deq = Q.dequant_group(d, s, n, gs, fmt, odt)
        assert torch.allclose(deq.float().cpu(), deq_ref, rtol=1e-2 if odt == torch.bfloat16 else 1e-6, atol=1e-6)


def test_ternary_kernels():
    torch.manual_seed(0)
    w = torch.randn(100, 333)
    t_ref = ternary.TernaryTensor.quantize(w)
    t = ternary.TernaryTensor.quantize(w.to(DEV))
    assert torch.allclose(t.scales.cpu(), t_ref.scales, rtol=1e-5)
    assert float((t.values().cpu() != t_ref.values()).float().mean()) < 1e-3   # |w| within rounding of the threshold
    assert torch.equal(Q.ternary_unpack(t.packed.cpu(), t.numel, 333), t.values().cpu().reshape(-1))
    pos, neg, zero = t.value_counts()
    v = t.values().cpu()
    assert (pos, neg, zero) == (int((v == 1).sum()), int((v == -1).sum()), int((v == 0).sum()))
    lin = nn.Linear(333, 100).to_device(DEV)
    lin.weight.data.copy_(w)
    tl = ternary.TernaryLinear.from_linear(lin)
    x = torch.randn(64, 333, device=DEV)
    want = x.float() @ tl.ternary_weight.dequantize().t() + lin.bias.detach().float()
    got = tl.forward(x)
    assert torch.allclose(got, want, rtol=2e-2, atol=2e-2 * float(want.abs().max()))


def test_rotor_quant_kernel():
    torch.manual_seed(0)
    for dim in (12, 64, 100):
        rq = quant.RotorQuant(dim, 4)
        x = torch.randn(37, dim)
        want = rq.quantize(x)
        got = rq.quantize(x.to(DEV)).cpu()
        close = (got - want).abs() < 1e-4
        assert float(close.float().mean()) > 0.995                            # rounding ties aside
        xb = x.to(DEV).to(torch.bfloat16)
        assert rq.quantize(xb).dtype == torch.bfloat16


def test_csr_spmm_kernel():
    torch.manual_seed(0)
    d = torch.randn(200, 300)
    d[d.abs() < 1.0] = 0
    sm = cp.SparseMatrix.from_dense(d.to(DEV), 0.0)
    b = torch.randn(300, 70, device=DEV)
    assert torch.allclose(sm.spmm(b, 70), d.to(DEV) @ b, rtol=1e-4, atol=1e-4)
    assert torch.equal(sm.to_dense().cpu(), d)


def test_int8_linear_and_quantized_model_gpu():
    torch.manual_seed(0)
    model = nn.Sequential().add(nn.Linear(256, 512)).add(nn.ReLU()).add(nn.Linear(512, 64)).to_device(DEV)
    x = torch.randn(100, 256, device=DEV)
    want = model(x).detach().float()
    scale = float(want.abs().max())
    il = int8.Int8Linear.from_linear(model.layers[0])
    y0 = il.forward(x)
    w0 = torch.nn.functional.linear(x, model.layers[0].weight.detach().float(), model.layers[0].bias.detach().float())
    assert float((y0 - w0).abs().max()) < 0.03 * float(w0.abs().max())
    for fmt, gs, tol in ((qz.QuantFormat.INT8, 256, 0.05), (qz.QuantFormat.NF4, 64, 0.3), (qz.QuantFormat.NVFP4, 16, 0.3), (qz.QuantFormat.BF16, 0, 0.02)):
        qm = qz.QuantizedModel.from_model(model, fmt, gs)
        got = qm.forward(x)
        assert float((got - want).abs().max()) < tol * scale
    a = torch.randint(0, 256, (64, 128), dtype=torch.int32).to(torch.uint8).to(DEV)
    b = torch.randint(-128, 128, (128, 48), dtype=torch.int32).to(torch.int8).to(DEV)
    assert torch.equal(int8.igemm(a, b, 64, 128, 48).cpu(), int8.igemm_scalar(a, b, 64, 128, 48))
