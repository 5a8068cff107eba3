"""Numerics of every sm_100a kernel against a plain PyTorch fp32 reference of the same op.

Shapes include tile multiples and deliberately odd sizes (the reference's own tests do the same:
rust-nn src/blas.rs:1196,1242,1644). Inputs come from a deterministic LCG like the reference's
(src/blas.rs:1182-1190).
"""
import math

import pytest
import torch

from rust_neural_network_b200.ops import gemm as G
from rust_neural_network_b200.ops import kernels as K
from rust_neural_network_b200.utils.lcg import lcg_tensor

pytestmark = pytest.mark.gpu
DEV = "cuda"


def rel_err(a, b):
    a, b = a.float(), b.float()
    return float((a - b).norm() / (b.norm() + 1e-12))


# ----------------------------------------------------------------------------- GEMM
@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (256, 512, 256), (100, 72, 40), (1000, 264, 520), (128, 10, 256), (4096, 1024, 512)])
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
def test_gemm_bf16_layouts(M, N, K, a_mn, b_mn):
    a = lcg_tensor((K, M) if a_mn else (M, K), seed=1).to(DEV).bfloat16()
    b = lcg_tensor((K, N) if b_mn else (N, K), seed=2).to(DEV).bfloat16()
    out = G.gemm(a, b, a_mn=a_mn, b_mn=b_mn)
    ref = G.gemm_ref(a, b, a_mn=a_mn, b_mn=b_mn, out_dtype=torch.float32)
    assert out.shape == (M, N) and out.dtype == torch.bfloat16
    assert rel_err(out, ref) < 1e-2


@pytest.mark.parametrize("bn", [64, 128, 256])
def test_gemm_tile_widths(bn):
    a = lcg_tensor((384, 320), seed=3).to(DEV).bfloat16()
    b = lcg_tensor((520, 320), seed=4).to(DEV).bfloat16()
    out = G.gemm(a, b, bn=bn, out_dtype=torch.float32)
    ref = G.gemm_ref(a, b, out_dtype=torch.float32)
    assert rel_err(out, ref) < 5e-3


@pytest.mark.parametrize("act", ["none", "relu", "gelu", "silu", "sigmoid"])
def test_gemm_epilogue(act):
    M, N, K_ = 300, 256, 192
    a = lcg_tensor((M, K_), seed=5).to(DEV).bfloat16()
    b = lcg_tensor((N, K_), seed=6).to(DEV).bfloat16()
    bias = lcg_tensor((N,), seed=7).to(DEV)
    res = lcg_tensor((M, N), seed=8).to(DEV).bfloat16()
    out, aux = G.gemm(a, b, bias=bias, act=act, residual=res, want_aux=True)
    ref, aux_ref = G.gemm_ref(a, b, bias=bias, act=act, residual=res, want_aux=True, out_dtype=torch.float32)
    assert rel_err(out, ref) < 1e-2
    assert rel_err(aux, aux_ref) < 1e-2
    # activation-gradient epilogue (the backward fusion)
    out2 = G.gemm(a, b, aux_in=aux, dact=act if act != "none" else "gelu", out_dtype=torch.float32)
    ref2 = G.gemm_ref(a, b, aux_in=aux, dact=act if act != "none" else "gelu", out_dtype=torch.float32)
    assert rel_err(out2, ref2) < 1e-2


def test_gemm_splitk_accumulate():
    # dW-shaped: small M,N, long K, fp32 accumulation into an existing buffer
    Kd, M, N = 8192, 256, 384
    a = lcg_tensor((Kd, M), seed=9).to(DEV).bfloat16()
    b = lcg_tensor((Kd, N), seed=10).to(DEV).bfloat16()
    acc = torch.ones(M, N, device=DEV)
    G.gemm(a, b, a_mn=True, b_mn=True, accumulate_into=acc)
    ref = 1.0 + a.float().t() @ b.float()
    assert rel_err(acc, ref) < 2e-3
    out = G.gemm(a, b, a_mn=True, b_mn=True, out_dtype=torch.float32)   # fresh fp32 output, auto split-K
    assert rel_err(out, ref - 1.0) < 2e-3


def test_gemm_batched():
    a = lcg_tensor((3, 200, 128), seed=11).to(DEV).bfloat16()
    b = lcg_tensor((3, 136, 128), seed=12).to(DEV).bfloat16()
    out = G.gemm(a, b, out_dtype=torch.float32)
    ref = a.float() @ b.float().transpose(1, 2)
    assert rel_err(out, ref) < 5e-3


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True)])
def test_gemm_tf32(a_mn, b_mn):
    M, N, K_ = 200, 136, 784
    a = lcg_tensor((K_, M) if a_mn else (M, K_), seed=13).to(DEV)
    b = lcg_tensor((K_, N) if b_mn else (N, K_), seed=14).to(DEV)
    bias = lcg_tensor((N,), seed=15).to(DEV)
    out = G.gemm(a, b, a_mn=a_mn, b_mn=b_mn, bias=bias, act="relu")
    ref = G.gemm_ref(a, b, a_mn=a_mn, b_mn=b_mn, bias=bias, act="relu")
    assert out.dtype == torch.float32
    assert rel_err(out, ref) < 2e-3


def test_gemm_k_edge_cases():
    a = lcg_tensor((1, 8), seed=16).to(DEV).bfloat16()
    b = lcg_tensor((1, 8), seed=17).to(DEV).bfloat16()
    out = G.gemm(a, b, out_dtype=torch.float32)
    assert rel_err(out, a.float() @ b.float().t()) < 1e-2


# ----------------------------------------------------------------------------- elementwise
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("op", ["relu", "gelu", "silu", "sigmoid", "tanh", "softplus", "exp", "abs", "square"])
def test_unary(op, dtype):
    x = lcg_tensor((37, 1001), seed=20).to(DEV).to(dtype) * 3
    y = K.unary(x, op)
    ref = K.unary_ref(x.float(), op)
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-5
    assert torch.allclose(y.float(), ref, atol=tol, rtol=tol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("op", ["add", "sub", "mul", "relu_bwd", "gelu_bwd", "silu_bwd", "mul_silu", "softplus_bwd"])
def test_binary(op, dtype):
    a = lcg_tensor((33, 513), seed=21).to(DEV).to(dtype)
    b = lcg_tensor((33, 513), seed=22).to(DEV).to(dtype)
    y = K.binary(a, b, op)
    ref = K.binary_ref(a.float(), b.float(), op)
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-5
    assert torch.allclose(y.float(), ref, atol=tol, rtol=tol)
    row = lcg_tensor((513,), seed=23).to(DEV).to(dtype)
    y2 = K.binary(a, row, "add")
    assert torch.allclose(y2.float(), a.float() + row.float(), atol=tol, rtol=tol)


def test_colsum_reduce_cast():
    x = lcg_tensor((1000, 300), seed=24).to(DEV)
    assert torch.allclose(K.colsum(x), x.sum(0), atol=1e-3, rtol=1e-4)
    assert torch.allclose(K.colsum(x.bfloat16()), x.bfloat16().float().sum(0), atol=1e-2, rtol=1e-3)
    assert math.isclose(float(K.reduce_all(x, "sum")), float(x.sum()), rel_tol=1e-4, abs_tol=1e-2)
    assert math.isclose(float(K.reduce_all(x, "sumsq")), float((x * x).sum()), rel_tol=1e-4)
    assert float(K.reduce_all(x, "max")) == float(x.max())
    assert float(K.reduce_all(x, "min")) == float(x.min())
    assert torch.equal(K.cast(x, torch.bfloat16), x.bfloat16())


@pytest.mark.parametrize("rows,cols", [(8192, 512), (1000, 264), (77, 40), (5, 2048), (65536, 1536), (3001, 8)])
def test_colsum_bf16_vector_path(rows, cols):
    torch.manual_seed(rows + cols)
    x = torch.randn(rows, cols, device=DEV).bfloat16()
    want = x.double().sum(0)
    assert float((K.colsum(x).double() - want).abs().max()) < 2e-4 * math.sqrt(rows) + 1e-3
    wide = torch.randn(rows, cols + 16, device=DEV).bfloat16()
    view = wide[:, 8:8 + cols]                        # strided rows, 16-byte aligned start
    acc = torch.ones(cols, device=DEV)
    K.colsum(view, out=acc)
    assert float((acc.double() - 1.0 - view.double().sum(0)).abs().max()) < 2e-4 * math.sqrt(rows) + 1e-3


@pytest.mark.parametrize("act", ["gelu", "silu", "relu"])
@pytest.mark.parametrize("rows,cols", [(8192, 2048), (1000, 264), (77, 40), (33, 20)])
def test_dact_colsum_matches_reference(rows, cols, act):
    torch.manual_seed(rows + cols)
    g = torch.randn(rows, cols, device=DEV).bfloat16()
    pre = (torch.randn(rows, cols, device=DEV) * 1.5).bfloat16()
    want = (g.float() * G.dact_ref(pre.float(), act)).bfloat16()
    acc = torch.full((cols,), 2.0, device=DEV)
    got, none = K.dact_colsum(g.clone(), pre, act, bias_grad=acc)
    assert none is None
    assert float((got.float() - want.float()).abs().max()) < 2e-2 * max(1.0, float(want.float().abs().max()))
    tol = 4e-2 * math.sqrt(rows) + 1e-2
    assert float((acc - 2.0 - want.float().sum(0)).abs().max()) < tol
    got2, db = K.dact_colsum(g.clone(), pre, act)
    assert torch.equal(got2, got) and float((db - want.float().sum(0)).abs().max()) < tol


def test_embedding():
    table = lcg_tensor((1000, 64), seed=25).to(DEV).bfloat16()
    ids = torch.randint(0, 1000, (4, 77), device=DEV)
    assert torch.equal(K.embedding_fwd(table, ids), table[ids])
    g = lcg_tensor((4, 77, 64), seed=26).to(DEV).bfloat16()
    gt = K.embedding_bwd(g, ids, 1000)
    ref = torch.zeros(1000, 64, device=DEV).index_add_(0, ids.view(-1), g.view(-1, 64).float())
    assert torch.allclose(gt, ref, atol=1e-3, rtol=1e-3)


def test_dropout_and_fake_quant():
    x = torch.ones(1 << 16, device=DEV)
    y = K.dropout_mask_apply(x, 0.25, seed=123)
    kept = float((y > 0).float().mean())
    assert abs(kept - 0.75) < 0.02
    assert torch.allclose(y[y > 0], torch.full_like(y[y > 0], 1 / 0.75))
    assert torch.equal(y, K.dropout_mask_apply(x, 0.25, seed=123))
    z = lcg_tensor((999,), seed=27).to(DEV) * 2
    s = 1.0 / 127
    assert torch.allclose(K.fake_quant(z, s, -128, 127), torch.clamp(torch.round(z / s), -128, 127) * s, atol=1e-6)


# ----------------------------------------------------------------------------- norms
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,d", [(64, 512), (1000, 384), (33, 129), (17, 2048), (1237, 2048), (301, 1536), (77, 3072), (130, 4096), (5000, 1024),
                                    (9, 1280)])
def test_layernorm(rows, d, dtype):
    x = (lcg_tensor((rows, d), seed=30) * 2 + 0.5).to(DEV).to(dtype)
    gamma = (lcg_tensor((d,), seed=31) + 1.5).to(DEV)
    beta = lcg_tensor((d,), seed=32).to(DEV)
    y, mean, rstd = K.layernorm_fwd(x, gamma, beta, 1e-5)
    ref = torch.nn.functional.layer_norm(x.float(), (d,), gamma, beta, 1e-5)
    tol = 3e-2 if dtype == torch.bfloat16 else 1e-4
    assert torch.allclose(y.float(), ref, atol=tol, rtol=tol)
    dy = lcg_tensor((rows, d), seed=33).to(DEV).to(dtype)
    dx, dg, db = K.layernorm_bwd(dy, x, gamma, mean, rstd)
    xr = x.float().requires_grad_(True); gr = gamma.clone().requires_grad_(True); br = beta.clone().requires_grad_(True)
    torch.nn.functional.layer_norm(xr, (d,), gr, br, 1e-5).backward(dy.float())
    assert rel_err(dx, xr.grad) < (2e-2 if dtype == torch.bfloat16 else 1e-4)
    assert rel_err(dg, gr.grad) < 1e-3
    assert rel_err(db, br.grad) < 1e-3


@pytest.mark.parametrize("rows,d", [(1000, 512), (77, 2048), (33, 384), (65, 129)])
def test_add_layernorm_fwd(rows, d):
    torch.manual_seed(d)
    x = torch.randn(rows, d, device=DEV).bfloat16(); r = torch.randn(rows, d, device=DEV).bfloat16()
    gamma = torch.rand(d, device=DEV) + 0.5; beta = torch.randn(d, device=DEV)
    s, y, mean, rstd = K.add_layernorm_fwd(x, r, gamma, beta, 1e-5)
    want_s = (x.float() + r.float()).bfloat16()
    assert torch.equal(s, want_s)
    ref = torch.nn.functional.layer_norm(want_s.float(), (d,), gamma, beta, 1e-5)
    assert torch.allclose(y.float(), ref, atol=3e-2, rtol=3e-2)
    assert torch.allclose(mean, want_s.float().mean(1), atol=1e-4) and torch.allclose(rstd, torch.rsqrt(want_s.float().var(1, unbiased=False) + 1e-5), rtol=1e-3)


def test_batchnorm():
    x = (lcg_tensor((64, 300), seed=34) * 2 + 1).to(DEV)
    gamma = (lcg_tensor((300,), seed=35) + 1.5).to(DEV); beta = lcg_tensor((300,), seed=36).to(DEV)
    rm = torch.zeros(300, device=DEV); rv = torch.ones(300, device=DEV)
    y, mean, rstd = K.batchnorm_fwd(x, gamma, beta, rm, rv, 1e-5, 0.1, True)
    bn = torch.nn.BatchNorm1d(300, eps=1e-5, momentum=0.1).to(DEV)
    with torch.no_grad():
        bn.weight.copy_(gamma); bn.bias.copy_(beta)
    xr = x.clone().requires_grad_(True)
    ref = bn(xr)
    assert torch.allclose(y, ref, atol=1e-4, rtol=1e-4)
    assert torch.allclose(rm, bn.running_mean, atol=1e-5) and torch.allclose(rv, bn.running_var, atol=1e-4)
    dy = lcg_tensor((64, 300), seed=37).to(DEV)
    dx, dg, db = K.batchnorm_bwd(dy, x, gamma, mean, rstd, True)
    ref.backward(dy)
    assert rel_err(dx, xr.grad) < 1e-4 and rel_err(dg, bn.weight.grad) < 1e-4 and rel_err(db, bn.bias.grad) < 1e-4


# ----------------------------------------------------------------------------- losses
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,V", [(64, 32000), (33, 1000), (7, 10)])
def test_ce_label(rows, V, dtype):
    logits = (lcg_tensor((rows, V), seed=40) * 4).to(DEV).to(dtype)
    labels = torch.randint(0, V, (rows,), device=DEV)
    loss, grad = K.ce_label(logits, labels)
    lr = logits.float().requires_grad_(True)
    ref = torch.nn.functional.cross_entropy(lr, labels)
    ref.backward()
    assert math.isclose(float(loss), float(ref), rel_tol=1e-4, abs_tol=1e-4)
    assert rel_err(grad, lr.grad) < (1e-2 if dtype == torch.bfloat16 else 1e-4)


def test_ce_dense_and_pointwise():
    logits = (lcg_tensor((32, 10), seed=41) * 3).to(DEV)
    labels = torch.randint(0, 10, (32,), device=DEV)
    onehot = torch.nn.functional.one_hot(labels, 10).float()
    loss, grad = K.ce_dense(logits, onehot)
    lr = logits.clone().requires_grad_(True)
    ref = torch.nn.functional.cross_entropy(lr, labels); ref.backward()
    assert math.isclose(float(loss), float(ref), rel_tol=1e-5, abs_tol=1e-5)
    assert rel_err(grad, lr.grad) < 1e-4
    pred = lcg_tensor((50, 7), seed=42).to(DEV); tgt = lcg_tensor((50, 7), seed=43).to(DEV)
    F = torch.nn.functional
    for kind, fn in [("mse", lambda p, t: F.mse_loss(p, t)), ("l1", lambda p, t: F.l1_loss(p, t)),
                     ("huber", lambda p, t: F.huber_loss(p, t, delta=0.3)),
                     ("bce_logits", lambda p, t: F.binary_cross_entropy_with_logits(p, t.abs().clamp(0, 1)))]:
        t_use = tgt.abs().clamp(0, 1) if kind == "bce_logits" else tgt
        l, g = K.pointwise_loss(pred, t_use, kind, delta=0.3)
        pr = pred.clone().requires_grad_(True)
        r = fn(pr, tgt); r.backward()
        assert math.isclose(float(l), float(r), rel_tol=1e-4, abs_tol=1e-5), kind
        assert rel_err(g, pr.grad) < 1e-4, kind
    prob = torch.sigmoid(pred); t01 = (tgt > 0).float()
    l, g = K.pointwise_loss(prob, t01, "bce")
    pr = prob.clone().requires_grad_(True)
    r = F.binary_cross_entropy(pr, t01); r.backward()
    assert math.isclose(float(l), float(r), rel_tol=1e-4) and rel_err(g, pr.grad) < 1e-4


# ----------------------------------------------------------------------------- optimizers
@pytest.mark.parametrize("torch_form", [0, 1])
def test_adam_matches_reference_forms(torch_form):
    n = 10007
    p0 = lcg_tensor((n,), seed=50); g = [lcg_tensor((n,), seed=51 + i) for i in range(3)]
    pd = p0.to(DEV).clone(); m = torch.zeros(n, device=DEV); v = torch.zeros(n, device=DEV)
    shadow = torch.empty(n, device=DEV, dtype=torch.bfloat16); step = torch.zeros(1, device=DEV)
    pc = p0.clone(); mc = torch.zeros(n); vc = torch.zeros(n); stepc = torch.zeros(1)
    for gi in g:
        K.adam_step(pd, gi.to(DEV), m, v, shadow, 1e-3, 0.9, 0.999, 1e-8, 0.0, torch_form, step)
        K.adam_step(pc, gi, mc, vc, None, 1e-3, 0.9, 0.999, 1e-8, 0.0, torch_form, stepc)
    assert float(step) == 3.0
    assert torch.allclose(pd.cpu(), pc, atol=1e-6, rtol=1e-5)
    assert torch.equal(shadow, pd.bfloat16())
    if torch_form:
        pt = torch.nn.Parameter(p0.clone()); opt = torch.optim.Adam([pt], lr=1e-3, eps=1e-8)
        for gi in g:
            pt.grad = gi.clone(); opt.step()
        assert torch.allclose(pd.cpu(), pt.detach(), atol=1e-6, rtol=1e-5)


def test_sgd_rmsprop_muon():
    n = 5001
    p0 = lcg_tensor((n,), seed=60); g1 = lcg_tensor((n,), seed=61); g2 = lcg_tensor((n,), seed=62)
    for name in ("sgd", "rmsprop", "muon"):
        pd = p0.to(DEV).clone(); pc = p0.clone()
        sd = torch.zeros(n, device=DEV); sc = torch.zeros(n)
        std = torch.zeros(1, device=DEV); stc = torch.zeros(1)
        seg = torch.tensor([[0, 1000], [1000, 1000], [1000, n]], dtype=torch.int64)
        for gi in (g1, g2):
            if name == "sgd":
                K.sgd_step(pd, gi.to(DEV), sd, None, 0.1, 0.9, std); K.sgd_step(pc, gi, sc, None, 0.1, 0.9, stc)
            elif name == "rmsprop":
                K.rmsprop_step(pd, gi.to(DEV), sd, None, 0.01, 0.99, 1e-8); K.rmsprop_step(pc, gi, sc, None, 0.01, 0.99, 1e-8)
            else:
                K.muon_rms_step(pd, gi.to(DEV), sd, None, seg.to(DEV), 0.02, 0.95); K.muon_rms_step(pc, gi, sc, None, seg, 0.02, 0.95)
        assert torch.allclose(pd.cpu(), pc, atol=1e-5, rtol=1e-4), name


# ----------------------------------------------------------------------------- attention
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("B,S,H,hd", [(2, 256, 2, 64), (1, 200, 3, 64), (2, 384, 2, 128), (1, 1024, 1, 64), (1, 130, 1, 128),
                                      (2, 200, 8, 64), (2, 136, 16, 128)])   # 256-row delta tiles that straddle two batches
def test_flash_forward_backward(B, S, H, hd, causal):
    torch.manual_seed(0)
    qkv = (torch.randn(B, S, 3, H, hd, device=DEV) * 0.8).bfloat16()
    q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]          # strided views of a fused buffer
    scale = 1.0 / math.sqrt(hd)
    o, lse = K.flash_fwd(q, k, v, scale, causal)
    qr, kr, vr = (t.float().detach().requires_grad_(True) for t in (q, k, v))
    ref = K.attention_ref(qr, kr, vr, scale, causal)
    assert rel_err(o, ref) < 1.5e-2
    s = (qr.permute(0, 2, 1, 3) @ kr.permute(0, 2, 1, 3).transpose(-1, -2)) * scale
    if causal:
        s = s.masked_fill(~torch.ones(S, S, dtype=torch.bool, device=DEV).tril(), float("-inf"))
    assert torch.allclose(lse, torch.logsumexp(s, -1), atol=2e-2, rtol=1e-2)
    do = (torch.randn(B, S, H, hd, device=DEV) * 0.5).bfloat16()
    dqkv = torch.empty_like(qkv)
    dq, dk, dv = K.flash_bwd(do, q, k, v, o, lse, scale, causal, dq=dqkv[:, :, 0], dk=dqkv[:, :, 1], dv=dqkv[:, :, 2])
    ref.backward(do.float())
    assert rel_err(dv, vr.grad) < 2e-2
    assert rel_err(dk, kr.grad) < 2e-2
    assert rel_err(dq, qr.grad) < 2e-2


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,cols,causal", [(64, 37, 0), (256, 1024, 0), (96, 48, 48), (8, 4099, 0)])
def test_softmax_rows_forward_backward(dtype, rows, cols, causal):
    """Row softmax kernel (scale, optional causal mask) against fp32 torch, forward and backward."""
    from rust_neural_network_b200.ops import functional as F
    torch.manual_seed(0)
    x = torch.randn(rows, cols, device="cuda").to(dtype).requires_grad_(True)
    w = torch.randn(rows, cols, device="cuda").to(dtype)
    y = F.softmax(x, 0.7, causal)
    y.backward(w)
    xr = x.detach().float().requires_grad_(True)
    s = xr * 0.7
    if causal:
        s = s.reshape(-1, causal, cols).masked_fill(~torch.ones(causal, cols, dtype=torch.bool, device="cuda").tril(), float("-inf")).reshape(rows, cols)
    ref = torch.softmax(s, -1)
    ref.backward(w.float())
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    assert torch.allclose(y.float(), ref, atol=tol, rtol=tol)
    assert torch.allclose(x.grad.float(), xr.grad, atol=tol * 4, rtol=tol * 4)


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("M,N,K", [(8192, 2048, 512), (5000, 1800, 192), (16384, 512, 2048)])
def test_gemm_cta_pair_tiles(M, N, K, a_mn, b_mn):
    """Shapes with enough 256 x 256 tiles to take the CTA-pair kernel (one MMA across two SMs), against the same product
    on single-CTA tiles (must agree to the last bit: same K order, same fp32 accumulation) and against fp32."""
    from rust_neural_network_b200 import _native as nv
    torch.manual_seed(M + N + K)
    a = torch.randn((K, M) if a_mn else (M, K), device="cuda").bfloat16()
    b = torch.randn((K, N) if b_mn else (N, K), device="cuda").bfloat16()
    bias = torch.randn(N, device="cuda")
    res = torch.randn(M, N, device="cuda").bfloat16()
    nv.set_gemm_pair(True, force=True)
    out = G.gemm(a, b, a_mn=a_mn, b_mn=b_mn, bias=bias, act="gelu", residual=res, bn=256)
    out32 = G.gemm(a, b, a_mn=a_mn, b_mn=b_mn, out_dtype=torch.float32, bn=256)
    nv.set_gemm_pair(False)
    one = G.gemm(a, b, a_mn=a_mn, b_mn=b_mn, bias=bias, act="gelu", residual=res, bn=256)
    one32 = G.gemm(a, b, a_mn=a_mn, b_mn=b_mn, out_dtype=torch.float32, bn=256)
    nv.set_gemm_pair(True)
    torch.cuda.synchronize(); nv.check_status()
    assert torch.equal(out, one) and torch.equal(out32, one32)
    ref = G.gemm_ref(a, b, a_mn=a_mn, b_mn=b_mn, out_dtype=torch.float32)
    assert rel_err(out32, ref) < 1e-5


def test_gemm_cta_pair_split_k_and_batch():
    from rust_neural_network_b200 import _native as nv
    torch.manual_seed(11)
    nv.set_gemm_pair(True, force=True)
    a = torch.randn(4096, 2048, device="cuda").bfloat16()           # dW-like: A, B MN-major, long K, split-K with fp32 atomics
    b = torch.randn(4096, 1024, device="cuda").bfloat16()
    acc = torch.zeros(2048, 1024, device="cuda")
    G.gemm(a, b, a_mn=True, b_mn=True, accumulate_into=acc, bn=256)
    ref = a.float().t() @ b.float()
    assert rel_err(acc, ref) < 1e-4
    ab = torch.randn(6, 1024, 256, device="cuda").bfloat16()
    bb = torch.randn(6, 2048, 256, device="cuda").bfloat16()
    out = G.gemm(ab, bb, out_dtype=torch.float32, bn=256)
    torch.cuda.synchronize(); nv.check_status()
    nv.set_gemm_pair(True)
    assert rel_err(out, ab.float() @ bb.float().transpose(1, 2)) < 1e-5


@pytest.mark.parametrize("M,N,K", [(4096, 1536, 512), (1000, 520, 256), (300, 2048, 128)])
def test_gemm_tma_store_epilogue_matches_plain_stores(M, N, K):
    """bf16 outputs (C and the saved pre-activation) through TMA stores, ragged edges included, against per-thread stores."""
    from rust_neural_network_b200 import _native as nv
    torch.manual_seed(M)
    a, b = torch.randn(M, K, device="cuda").bfloat16(), torch.randn(N, K, device="cuda").bfloat16()
    bias, res = torch.randn(N, device="cuda"), torch.randn(M, N, device="cuda").bfloat16()
    outs = []
    for on in (True, False):
        nv.set_gemm_tma_store(on)
        y, aux = G.gemm(a, b, bias=bias, act="gelu", residual=res, want_aux=True)
        outs.append((y.clone(), aux.clone()))
    nv.set_gemm_tma_store(True)
    torch.cuda.synchronize(); nv.check_status()
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])
    ref, _ = G.gemm_ref(a, b, bias=bias, act="gelu", residual=res, want_aux=True, out_dtype=torch.float32)
    assert rel_err(outs[0][0], ref) < 1e-2


@pytest.mark.parametrize("rows,d", [(1000, 512), (4096, 1024), (300, 768), (64, 2048)])
def test_layernorm_bwd_with_fused_column_sums(rows, d):
    """The backward that also returns the column sums of the residual gradient and of its own output (the bias gradients
    on either side of a pre-norm LayerNorm) against the plain backward plus two column sums; d = 2048 takes the fallback."""
    torch.manual_seed(rows + d)
    x = torch.randn(rows, d, device=DEV).bfloat16()
    dy, dres = torch.randn(rows, d, device=DEV).bfloat16(), torch.randn(rows, d, device=DEV).bfloat16()
    g = torch.randn(d, device=DEV)
    _, mean, rstd = K.layernorm_fwd(x, g, torch.zeros(d, device=DEV), 1e-5)
    s_res, s_dx = torch.ones(d, device=DEV), torch.full((d,), 2.0, device=DEV)           # accumulators: added to
    dx, dg, db = K.layernorm_bwd(dy, x, g, mean, rstd, dres=dres, sum_dres=s_res, sum_dx=s_dx)
    dx0, dg0, db0 = K.layernorm_bwd(dy, x, g, mean, rstd, dres=dres)
    assert torch.equal(dx, dx0)
    assert torch.allclose(dg, dg0, rtol=1e-3, atol=1e-2) and torch.allclose(db, db0, rtol=1e-3, atol=1e-2)
    assert torch.allclose(s_res - 1.0, dres.float().sum(0), rtol=1e-3, atol=2e-2)
    # the fused sum is taken before the bf16 rounding of dx, the reference after it
    assert torch.allclose(s_dx - 2.0, dx0.float().sum(0), rtol=1e-2, atol=0.5)


def test_gemm_ragged_groups():
    """Batched GEMM over ragged groups (the tokens routed to each expert): row tiles past `m_valid` are skipped, the K loop
    of a weight-gradient product stops at `k_valid` rounded up to 128, and skipped tiles may hold anything."""
    from rust_neural_network_b200 import _native as nv
    torch.manual_seed(21)
    E, cap, d, hid = 6, 640, 256, 384
    counts = torch.tensor([640, 0, 130, 128, 511, 1], dtype=torch.int32, device=DEV)
    x = torch.randn(E, cap, d, device=DEV).bfloat16()
    for e in range(E):
        x[e, int(counts[e]):] = 0                                   # rows past the count are zero, as a dispatch buffer is
    w = torch.randn(E, hid, d, device=DEV).bfloat16()
    bias = torch.randn(E, hid, device=DEV)
    out = torch.full((E, cap, hid), float("nan"), device=DEV, dtype=torch.bfloat16)
    G.gemm(x, w, bias=bias, act="silu", out=out, m_valid=counts)
    ref = G.gemm_ref(x, w, bias=bias, act="silu", out_dtype=torch.float32)
    for e in range(E):
        n = int(counts[e]); tiles = (n + 127) // 128 * 128
        assert rel_err(out[e, :tiles], ref[e, :tiles]) < 1e-2 or tiles == 0
        assert bool(torch.isnan(out[e, tiles:]).all())              # skipped tiles were not touched
    # weight gradient: dy^T h over the rows in use; rows past the computed tiles hold NaN on purpose
    dy = torch.randn(E, cap, hid, device=DEV).bfloat16()
    for e in range(E):
        dy[e, int(counts[e]):] = 0
    hbuf = out.clone()                                               # NaN in the skipped tiles
    dW = G.gemm(dy, hbuf, a_mn=True, b_mn=True, out_dtype=torch.float32, k_valid=counts)       # [E, hid(dy cols), hid]
    torch.cuda.synchronize(); nv.check_status()
    assert bool(torch.isfinite(dW).all())
    h_clean = torch.nan_to_num(hbuf.float(), nan=0.0)
    refW = dy.float().transpose(1, 2) @ h_clean
    assert rel_err(dW, refW) < 1e-2
    assert float(dW[1].abs().max()) == 0.0                          # an empty group contributes nothing


@pytest.mark.parametrize("rows,cols,sliced", [(1000, 512, True), (4096, 2048, True), (300, 64, False), (77, 24, True)])
def test_gate_forward_backward_on_column_slices(rows, cols, sliced):
    """y * silu(z) and its two gradients in one pass each, with z (and g) taken as column slices of a wider matrix."""
    torch.manual_seed(rows)
    wide = torch.randn(rows, 2 * cols, device=DEV).bfloat16()
    z = wide[:, cols:] if sliced else wide[:, cols:].contiguous()
    y = torch.randn(rows, cols, device=DEV).bfloat16()
    gw = torch.randn(rows, cols + 8, device=DEV).bfloat16()
    g = gw[:, :cols] if sliced else gw[:, :cols].contiguous()
    out = K.gate_fwd(y, z)
    dy, dz = K.gate_bwd(g, y, z)
    yf, zf, gf = (t.float().requires_grad_(True) for t in (y, z, g))
    ref = yf * torch.nn.functional.silu(zf)
    ref.backward(gf.detach())
    assert rel_err(out, ref) < 5e-3
    assert rel_err(dy, yf.grad) < 5e-3 and rel_err(dz, zf.grad) < 5e-3
    o3 = K.gate_fwd(y.view(1, rows, cols), z.view(1, rows, cols) if not sliced else wide.view(1, rows, 2 * cols)[:, :, cols:])
    assert torch.equal(o3.view(rows, cols), out)
