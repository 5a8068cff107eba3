"""CPU tests of the low-precision / compression modules (the PyTorch restatements of the kernels'
arithmetic, which the GPU tests then use as oracles)."""
import math
import random

import pytest
import torch

from rust_neural_network_b200 import nn, int8, quantize as qz, quant, ternary, compression as cp
from rust_neural_network_b200.loss import MSELoss
from rust_neural_network_b200.ops import quant_kernels as Q


def test_int8_weights_roundtrip_and_ratio():
    torch.manual_seed(0)
    w = torch.randn(16, 32)
    q = int8.Int8Weights.quantize(w)
    assert q.data.dtype == torch.int8 and tuple(q.data.shape) == (16, 32) and q.scales.shape == (16,)
    assert torch.allclose(q.scales, w.abs().amax(-1) / 127)
    assert q.quantization_error(w) < float(w.abs().max()) / 127
    assert q.mem_bytes() == 16 * 32 + 16 * 4 and q.compression_ratio() > 3.5
    z = int8.Int8Weights.quantize(torch.zeros(2, 4))
    assert z.scales.tolist() == [1.0, 1.0] and int(z.data.abs().sum()) == 0


def test_int8_linear_close_to_fp32_and_reference_mode():
    torch.manual_seed(0)
    lin = nn.Linear(32, 8)
    lin.bias.data.normal_()
    x = torch.randn(5, 32)
    want = lin(x).detach()
    got = int8.Int8Linear.from_linear(lin).forward(x)
    assert tuple(got.shape) == (5, 8) and float((got - want).abs().max()) < 0.05 * float(want.abs().max()) + 0.05
    ref_mode = int8.Int8Linear.from_linear(lin, mode="reference").forward(x)
    # hand evaluation of the reference's formula for one output
    w = int8.Int8Weights.quantize(lin.weight)
    s = float(w.scales[3])
    acc = sum(int(max(-128, min(127, math.floor(abs(float(x[2, k])) / s + 0.5) * (1 if x[2, k] >= 0 else -1)))) * int(w.data[3, k]) for k in range(32))
    assert float(ref_mode[2, 3]) == pytest.approx(acc * s * s + float(lin.bias[3]), rel=1e-4, abs=1e-4)


def test_igemm_matches_scalar_oracle():
    g = torch.Generator().manual_seed(1)
    a = torch.randint(0, 256, (7, 40), generator=g, dtype=torch.int32).to(torch.uint8)
    b = torch.randint(-128, 128, (40, 9), generator=g, dtype=torch.int32).to(torch.int8)
    out = int8.igemm(a, b, 7, 40, 9)
    want = torch.zeros(7, 9, dtype=torch.int64)
    for i in range(7):
        for j in range(9):
            want[i, j] = sum(int(a[i, k]) * int(b[k, j]) for k in range(40))
    assert out.dtype == torch.int32 and torch.equal(out.long(), want)


@pytest.mark.parametrize("fmt,tol", [(qz.QuantFormat.FP16, 1e-3), (qz.QuantFormat.BF16, 1e-2), (qz.QuantFormat.INT8, 0.01),
                                     (qz.QuantFormat.INT4, 0.12), (qz.QuantFormat.NF4, 0.12), (qz.QuantFormat.NVFP4, 0.15),
                                     (qz.QuantFormat.GGUF_Q4, 0.12), (qz.QuantFormat.GGUF_Q4K, 0.12), (qz.QuantFormat.GGUF_Q8, 0.01)])
def test_quant_formats_roundtrip(fmt, tol):
    torch.manual_seed(0)
    t = torch.randn(6, 50)
    q = qz.quantize(t, fmt, 32)
    d = q.dequantize()
    assert tuple(d.shape) == (6, 50)
    assert q.quantization_error(t) < tol * float(t.abs().max())
    assert q.compression_ratio() > 0.8 * fmt.compression_ratio() * (0.75 if fmt.bits() <= 8 else 1.0)
    assert fmt.bits() in (4, 8, 16)


def test_quant_reference_vectors():
    # INT8, whole tensor as one group: scale 0.9/127 (src/quantize.rs int8_roundtrip)
    t = torch.tensor([[0.1, 0.5, -0.3], [0.8, -0.9, 0.0]])
    q = qz.QuantizedTensor.quantize(t, qz.QuantFormat.INT8, 0)
    assert q.group_size == 6 and q.scales.tolist() == pytest.approx([0.9 / 127])
    assert q.data.view(torch.int8).tolist() == [14, 71, -42, 113, -127, 0]
    # INT4 nibble order: low nibble first, two's-complement nibbles
    q4 = qz.QuantizedTensor.quantize(torch.tensor([7.0, -7.0, 1.0, 0.0]), qz.QuantFormat.INT4, 0)
    assert q4.scales.tolist() == [1.0] and q4.data.tolist() == [0x97, 0x01]
    # NF4: normalised by max|x|; +-1 map to codes 15 / 0
    qn = qz.QuantizedTensor.quantize(torch.tensor([2.0, -2.0, 0.0, 1.0]), qz.QuantFormat.NF4, 0)
    assert qn.scales.tolist() == [2.0] and qn.data.tolist() == [0x0F, 0xC7]
    # NVFP4: scale max/6; sign bit 8
    qf = qz.QuantizedTensor.quantize(torch.tensor([6.0, -3.0, 0.5, -0.2]), qz.QuantFormat.NVFP4, 0)
    assert qf.scales.tolist() == [1.0] and qf.data.tolist() == [0xD7, 0x01 | (0x8 << 4)]
    assert qf.dequantize().tolist() == [6.0, -3.0, 0.5, -0.0]
    # Q4_0: negative scale max/-8, blocks of at most 32
    qg = qz.QuantizedTensor.quantize(torch.arange(40, dtype=torch.float32) - 20.0, qz.QuantFormat.GGUF_Q4, 64)
    assert qg.group_size == 32 and qg.scales.numel() == 2 and float(qg.scales[0]) == pytest.approx(-2.5)
    assert qg.data.numel() == 16 + 4
    # odd group size: one pad nibble per group
    qo = qz.QuantizedTensor.quantize(torch.ones(6), qz.QuantFormat.INT4, 3)
    assert qo.data.numel() == 4 and torch.allclose(qo.dequantize(), torch.ones(6))
    assert qz.QuantFormat.NF4.name_str() == "NF4 (NormalFloat 4-bit)" and qz.QuantFormat.INT8.compression_ratio() == 4.0


def test_quantized_linear_and_model():
    torch.manual_seed(0)
    model = nn.Sequential().add(nn.Linear(16, 32)).add(nn.ReLU()).add(nn.Linear(32, 4))
    x = torch.randn(3, 16)
    want = model(x).detach()
    for fmt in (qz.QuantFormat.INT8, qz.QuantFormat.NF4, qz.QuantFormat.BF16):
        qm = qz.QuantizedModel.from_model(model, fmt, 16)
        assert len(qm.layers()) == 2 and qm.compression_ratio() > 1.5
        got = qm.forward(x)
        assert float((got - want).abs().max()) < 0.25 * float(want.abs().max()) + 0.05
    ql = qz.QuantizedLinear.from_linear(model.layers[0], qz.QuantFormat.INT8, 16)
    assert ql._rowwise_int8() and tuple(ql.forward(x).shape) == (3, 32)


def test_rotor_and_rotorquant():
    rng = random.Random(42)
    for _ in range(20):
        R = torch.tensor(quant.Rotor.random(rng).rotation_matrix())
        assert torch.allclose(R @ R.T, torch.eye(3), atol=1e-5) and float(torch.det(R)) == pytest.approx(1.0, abs=1e-4)
    r = quant.Rotor.random(random.Random(7))
    x = [0.0, 0.3, -1.7, 2.1, 0.0, 0.0, 0.0, 0.0]
    back = r.inv_sandwich(r.sandwich(x))
    assert all(abs(a - b) < 1e-6 for a, b in zip(x, back))
    rq = quant.RotorQuant.with_seed(12, 4, 123)
    data = torch.tensor([i * 0.37 - 1.5 for i in range(12)])
    q = rq.quantize(data)
    assert float((q - data).abs().max()) < 0.15 * float(data.max() - data.min())
    assert rq.padded_dim == 12 and len(rq.rotors) == 4 and rq.qmax() == 7.0 and rq.parameters() == []
    rq2 = quant.RotorQuant(10, 8)                      # dim not a multiple of 3: padded to 12
    y = rq2.forward(torch.randn(4, 10))
    assert tuple(y.shape) == (4, 10) and rq2.padded_dim == 12
    assert torch.equal(rq2.quantize(torch.zeros(2, 10)), torch.zeros(2, 10))
    e8 = float((quant.RotorQuant(12, 8).quantize(data) - data).abs().max())
    assert e8 < float((q - data).abs().max())
    with pytest.raises(ValueError):
        quant.RotorQuant(4, 1)
    with pytest.raises(ValueError):
        rq.quantize(torch.zeros(5))


def test_ternary_tensor_and_linear():
    vals = [1, -1, 0, 1, 0, 0, -1, -1, 1, 0, 1, -1, 0, 1, -1, 0, 1, -1, 0]
    assert ternary.unpack_ternary(ternary.pack_ternary(vals), len(vals)) == vals
    t = torch.tensor([[0.5, -0.3, 0.01, -0.8], [0.6, -0.02, 0.9, -0.4]])
    q = ternary.TernaryTensor.quantize(t)
    assert q.values().tolist() == [[1.0, -1.0, 0.0, -1.0], [1.0, 0.0, 1.0, -1.0]]
    assert q.scales.tolist() == pytest.approx([0.4025, 0.48])
    assert q.packed.tolist() == ternary.pack_ternary([1, -1, 0, -1, 1, 0, 1, -1])
    assert q.value_counts() == (3, 3, 2) and q.sparsity() == pytest.approx(2 / 8)
    torch.manual_seed(0)
    big = ternary.ternarize(torch.randn(64, 128))
    assert big.compression_ratio() > 10.0 and 0.2 < big.sparsity() < 0.7
    assert big.quantization_error(big.dequantize()) == 0.0
    lin = nn.Linear(128, 16)
    tl = ternary.TernaryLinear.from_linear(lin)
    x = torch.randn(4, 128)
    y = tl.forward(x)
    want = x @ tl.ternary_weight.dequantize().t() + lin.bias.detach()
    assert tuple(y.shape) == (4, 16) and torch.allclose(y, want, atol=1e-4)
    model = nn.Sequential().add(nn.Linear(32, 64)).add(nn.ReLU()).add(nn.Linear(64, 8))
    tm = ternary.TernaryModel.from_model(model)
    assert len(tm.layers) == 2 and tm.compression_ratio() > 6.0 and 0.0 < tm.avg_sparsity() < 1.0
    assert tuple(tm.forward_first_layer(torch.randn(2, 32)).shape) == (2, 64) and tuple(tm.forward(torch.randn(2, 32)).shape) == (2, 8)


def test_compression_toolkit():
    torch.manual_seed(0)
    ws = cp.SharedWeights(64, 64, 4)
    assert ws.compression_ratio() > 3.5 and tuple(ws.forward(torch.randn(2, 64)).shape) == (2, 64) and ws.param_count() == 64 * 64 + 64
    d = torch.tensor([[1.0, 0.0, 0.0, 2.0], [0.0, 0.0, 0.0, 0.0], [0.05, -3.0, 0.0, 0.0]])
    sm = cp.SparseMatrix.from_dense(d, 0.1)
    assert sm.nnz == 3 and sm.row_ptrs.tolist() == [0, 2, 2, 3] and sm.col_indices.tolist() == [0, 3, 1]
    assert sm.sparsity() == pytest.approx(0.75)
    dd = d.clone(); dd[2, 0] = 0.0
    assert torch.equal(sm.to_dense(), dd)
    b = torch.randn(4, 5)
    assert torch.allclose(sm.spmm(b.reshape(-1), 5), dd @ b, atol=1e-6)
    ld = cp.LayerDropper(2, 0.1)
    x = torch.ones(4)
    assert ld.should_skip(0, x, x * 1.01) and not ld.should_skip(1, x, x * 2)
    assert ld.avg_skip_rate() == pytest.approx(0.25) and ld.estimated_speedup() == pytest.approx(1 / 0.75)
    kt = cp.KnowledgeTransfer(nn.Linear(6, 8), nn.Linear(6, 8), 8, 8)
    assert kt.transfer_loss(torch.randn(3, 6)) >= 0.0
    table = torch.randn(50, 16)
    ce = cp.CompressedEmbedding.from_table(table, 4)
    assert ce.compression_ratio() == pytest.approx(50 * 16 / (50 * 4 + 4 * 16)) and tuple(ce.lookup(3).shape) == (1, 16)
    assert torch.allclose(ce.lookup_batch([1, 7]), ce.reconstruct()[[1, 7]], atol=1e-4) and ce.mem_bytes() == (200 + 64) * 4
    svd = cp.CompressedEmbedding.from_table_svd(table, 16)
    assert torch.allclose(svd.reconstruct(), table, atol=1e-3)
    ps = cp.ProgressiveShrinking(0.5, 10, 2)
    vals = [ps.step() for _ in range(10)]
    assert vals[0] == 0.0 and vals[1] == 0.0 and vals[5] == pytest.approx(0.25) and vals[-1] == 0.5 and ps.is_done()
    pr = ps.apply_soft_prune(torch.arange(1.0, 11.0))
    assert int((pr == 0).sum()) == 6                        # threshold = sorted[5], pruned with <=
    w = torch.tensor([[3.0, 0.0], [0.1, 0.0], [1.0, 1.0], [0.0, 0.2]])
    pw, kept = cp.StructuredPruner.prune_channels(w, 0.5)
    assert kept == [2, 0] and tuple(pw.shape) == (2, 2)
    lin = nn.Linear(2, 4)
    lin.weight.data.copy_(w)
    nl, kept2 = cp.StructuredPruner.prune_linear(lin, 0.5)
    assert kept2 == [2, 0] and tuple(nl.weight.shape) == (2, 2) and nl.bias.numel() == 2 and nl.out_features == 2
    assert cp.CompressionStrategy.Quantize(8).size_factor() == 4.0 and cp.CompressionStrategy.Prune(0.5).size_factor() == 2.0
    assert cp.CompressionStrategy.LowRank(4).size_factor() == 4.0 and cp.CompressionStrategy.None_().size_factor() == 1.0


def test_mixed_sparsity_and_automl():
    torch.manual_seed(0)
    model = nn.Sequential().add(nn.Linear(8, 16)).add(nn.ReLU()).add(nn.Linear(16, 4))
    x, y = torch.randn(10, 8), torch.randn(10, 4)
    before = [p.detach().clone() for p in model.parameters()]
    ms = cp.MixedSparsity.analyze(model, x, y, MSELoss())
    assert len(ms.layer_sparsity) == 4 and all(0.05 <= s <= 0.9 for s in ms.layer_sparsity) and ms.sparsity_for_layer(99) == 0.5
    assert all(torch.equal(a, b.detach()) for a, b in zip(before, model.parameters()))      # parameters restored
    rec = cp.automl_search(model, x, y, MSELoss(), 2.0)
    assert len(rec.strategies) >= 1 and rec.compression_ratio >= 1.0 and rec.accuracy_retention <= 1.0
    assert rec.strategies[0].kind == "none"                  # score 1.0 ties resolve to the last maximum... which is "none" only if nothing else reaches 1.0
