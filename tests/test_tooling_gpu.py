"""GPU tests of the BLAS / SIMD / fused / compiled / GPU-backend surfaces and the HBM tier of the store."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

from rust_neural_network_b200 import blas, compiled, fused, gpu, nn, offload, simd

DEV = "cuda"


@pytest.mark.parametrize("m,n", [(1000, 4096), (37, 129), (4096, 1000), (8, 100000)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gemv_both_orientations(m, n, dtype):
    torch.manual_seed(m + n)
    a = torch.randn(m, n, device=DEV).to(dtype)
    x, xt = torch.randn(n, device=DEV), torch.randn(m, device=DEV)
    y = torch.randn(m, device=DEV)
    want = 1.5 * (a.double() @ x.double()) - 0.5 * y.double()
    blas.sgemv(blas.Transpose.NoTrans, m, n, 1.5, a, n, x, 1, -0.5, y, 1)
    assert torch.allclose(y.double(), want, rtol=1e-4, atol=1e-3 * math.sqrt(n))
    yt = torch.zeros(n, device=DEV)
    blas.sgemv(blas.Transpose.Trans, m, n, 2.0, a, n, xt, 1, 0.0, yt, 1)
    assert torch.allclose(yt.double(), 2.0 * (a.double().t() @ xt.double()), rtol=1e-4, atol=1e-3 * math.sqrt(m))


def test_blas_level1_and_sgemm_gpu():
    torch.manual_seed(0)
    x, y = torch.randn(100003, device=DEV), torch.randn(100003, device=DEV)
    assert float(blas.sdot(100003, x, 1, y, 1)) == pytest.approx(float((x.double() * y.double()).sum()), rel=1e-4, abs=1e-2)
    assert float(blas.snrm2(100003, x)) == pytest.approx(float(x.double().norm()), rel=1e-5)
    assert float(blas.sdot(50000, x, 2, y, 2)) == pytest.approx(float((x[::2][:50000].double() * y[::2][:50000].double()).sum()), rel=1e-4, abs=1e-2)
    y0 = y.clone()
    blas.saxpy(100003, 0.25, x, y)
    assert torch.allclose(y, y0 + 0.25 * x, atol=1e-6)
    blas.sscal(100003, 2.0, y)
    assert torch.allclose(y, 2 * (y0 + 0.25 * x), atol=1e-5)
    a, b = torch.randn(300, 200, device=DEV), torch.randn(200, 160, device=DEV)
    c = torch.ones(300, 160, device=DEV)
    blas.sgemm(blas.Transpose.NoTrans, blas.Transpose.NoTrans, 300, 160, 200, 2.0, a, 200, b, 160, 0.5, c, 160)
    want = 2.0 * a @ b + 0.5
    assert float((c - want).abs().max()) < 2e-2 * float(want.abs().max())          # TF32 products
    ct = torch.zeros(300, 160, device=DEV)
    blas.sgemm(blas.Transpose.Trans, blas.Transpose.Trans, 300, 160, 200, 1.0, a.t().contiguous(), 300, b.t().contiguous(), 200, 0.0, ct, 160)
    assert float((ct - a @ b).abs().max()) < 2e-2 * float((a @ b).abs().max())


def test_simd_and_fused_gpu():
    a, b = torch.randn(10000, device=DEV), torch.randn(10000, device=DEV)
    assert torch.allclose(simd.simd_add(a, b), a + b) and torch.allclose(simd.simd_mul(a, b), a * b)
    assert torch.equal(simd.simd_relu(a), torch.relu(a)) and torch.allclose(simd.simd_scale(a, 3.0), 3 * a)
    assert float(simd.simd_sum(a)) == pytest.approx(float(a.double().sum()), abs=1e-2) and "sm_" in simd.simd_features()
    x, w, bias = torch.randn(64, 256, device=DEV), torch.randn(128, 256, device=DEV), torch.randn(128, device=DEV)
    for act, ref in ((fused.FusedActivation.ReLU, torch.relu), (fused.FusedActivation.Sigmoid, torch.sigmoid), (fused.FusedActivation.None_, lambda t: t)):
        got = fused.fused_linear(x, w, bias, act)
        want = ref(x @ w.t() + bias)
        assert float((got - want).abs().max()) < 3e-2 * max(float(want.abs().max()), 1.0)
    logits = torch.randn(500, 16, device=DEV)
    idx, wts = fused.sparse_topk_route(logits, 500, 16, 4)
    vals, ti = torch.topk(logits, 4, -1)
    assert torch.equal(idx.view(500, 4).sort(-1).values, ti.sort(-1).values)
    assert torch.allclose(wts.view(500, 4).sort(-1).values, torch.softmax(vals, -1).sort(-1).values, atol=1e-5)


def test_compiled_mlp_graph_matches_eager():
    dims = [(16, 64), (64, 64), (64, 8)]
    g = torch.Generator().manual_seed(0)
    x, y = torch.randn(32, 16, generator=g), torch.randn(32, 8, generator=g)
    cg = compiled.CompiledMLP(dims, 32, 0.01, device=DEV)
    ce = compiled.CompiledMLP(dims, 32, 0.01, device="cpu")
    lg = [cg.step(x, y) for _ in range(20)]
    le = [ce.step(x, y) for _ in range(20)]
    assert cg.trainer._graph is not None and cg.trainer.launches_per_step > 0
    assert lg[0] == pytest.approx(le[0], rel=2e-2)          # the graph's warm-up steps left no trace in the weights
    assert lg[-1] == pytest.approx(le[-1], rel=0.1) and lg[-1] < 0.7 * lg[0]


def test_gpu_backend_surface():
    g = gpu.gpu()
    assert gpu.has_gpu() and g is not None and gpu.active_backend() is gpu.GpuBackendKind.Nvidia
    a, b = torch.randn(70, 50), torch.randn(50, 30)
    tol = 2e-2 * float((a @ b).abs().max())
    assert float((gpu.gpu_matmul(a, b).cpu() - a @ b).abs().max()) < tol
    c = torch.randn(70, 30)
    assert float((g.matmul_ab(a, b, 0.5, 2.0, c).cpu() - (0.5 * a @ b + 2 * c)).abs().max()) < tol
    w, bias = torch.randn(30, 50), torch.randn(30)
    assert float((gpu.gpu_linear(a, w, bias, True).cpu() - torch.relu(a @ w.t() + bias)).abs().max()) < tol
    for d in (32, 64, 100, 200):
        q, k, v = torch.randn(300, d), torch.randn(300, d), torch.randn(300, d)
        want = torch.softmax(q @ k.t() / math.sqrt(d), -1) @ v
        got = gpu.gpu_attention(q, k, v, 1 / math.sqrt(d)).cpu()
        assert tuple(got.shape) == (300, d) and float((got - want).abs().max()) < 3e-2
    t = torch.tensor([-1.0, 0.5])
    assert torch.equal(gpu.gpu_relu(t).cpu(), torch.tensor([0.0, 0.5])) and torch.allclose(g.activation(t, 1).cpu(), torch.sigmoid(t))
    assert torch.equal(gpu.gpu_add(t, t).cpu(), 2 * t) and torch.equal(gpu.gpu_mul(t, t).cpu(), t * t)
    out, used = gpu.kernel_matmul(a, b)
    assert used is gpu.GpuBackendKind.Nvidia and float((out - a @ b).abs().max()) < tol


def test_tiered_store_gpu_tier(tmp_path):
    cfg = offload.OffloadConfig().with_ssd_dir(str(tmp_path)).with_gpu_budget_gb(1.0, DEV)
    cfg.gpu_budget_bytes = 8000 + 10
    cfg.ram_budget_bytes = 4000 + 10
    store = offload.TieredStore(cfg)
    for i in range(4):
        store.insert(f"t{i}", torch.full((1000,), float(i), device=DEV))
    tiers = [store.tensors[f"t{i}"].tier() for i in range(4)]
    assert tiers == [offload.MemoryTier.Ssd, offload.MemoryTier.Ram, offload.MemoryTier.Gpu, offload.MemoryTier.Gpu]
    assert store.gpu_usage() == 8000 and store.ram_usage() == 4000
    t0 = store.get("t0", device=DEV)
    assert t0.is_cuda and float(t0.sum()) == 0.0 and store.tensors["t0"].tier() == offload.MemoryTier.Gpu
    assert store.gpu_usage() <= cfg.gpu_budget_bytes and store.ram_usage() <= cfg.ram_budget_bytes
    for i in range(4):
        assert float(store.get(f"t{i}", device=DEV)[0]) == float(i)
    model = nn.Sequential().add(nn.Linear(32, 32)).to_device(DEV)
    x = torch.randn(4, 32, device=DEV)
    want = model(x).detach().float().clone()
    om = offload.OffloadModel(model, offload.OffloadConfig().with_ssd_dir(str(tmp_path / "m")))
    om.offload()
    assert torch.allclose(om.forward(x).float(), want, atol=1e-5)
