"""gpu_kernels.py, one test per behaviour of rust-nn src/gpu_kernels.rs:780-970 that has a meaning on a B200-only
build: backend detection, the tile configuration, kernel_matmul, the embedded kernel source, the report. The
reference's AMD and Apple kernels have no counterpart: their names and tile descriptions stay, with a one-line source."""
import os

import pytest
import torch

from rust_neural_network_b200 import gpu_kernels as K
from rust_neural_network_b200.gpu import GpuBackendKind as B, TileConfig


def test_detect_backend_returns_a_valid_kind():
    assert K.detect_backend() in (B.Nvidia, B.Cpu)
    assert (K.detect_backend() == B.Nvidia) == torch.cuda.is_available()


def test_tile_config_nvidia():
    c = TileConfig.nvidia()
    assert c.bm >= 64 and c.bn >= 64 and c.warp_size == 32 and c.shared_mem_bytes() > 0
    assert c.bm == 128 and c.bk * 2 == 128                          # one 128-byte swizzle row of bf16 per K block


def test_other_vendors_keep_their_descriptive_tiles():
    assert TileConfig.amd().warp_size == 64 and TileConfig.amd().bk >= 32      # wavefronts are 64 lanes
    assert TileConfig.apple().bm >= 32 and TileConfig.apple().bk >= 8


def test_arithmetic_intensity_is_positive():
    for b in (B.Nvidia, B.Amd, B.Apple, B.Cpu):
        assert TileConfig.for_backend(b).arithmetic_intensity() > 0.0
    nv = TileConfig.nvidia()                                          # the reference's formula: bm*bn over the bytes of one k-slice
    assert nv.arithmetic_intensity() == pytest.approx(128 * 256 / ((128 * 64 + 64 * 256) * 2))


def test_kernel_matmul_values():
    a = torch.tensor([[1.0, 2.0], [3.0, 4.0]])
    b = torch.tensor([[5.0, 6.0], [7.0, 8.0]])
    c, used = K.kernel_matmul(a, b)
    assert used in (B.Nvidia, B.Cpu)
    assert c.reshape(-1).tolist() == pytest.approx([19.0, 22.0, 43.0, 50.0], abs=1e-3)


def test_kernel_matmul_with_an_explicit_backend():
    c, used = K.kernel_matmul_with_backend(torch.ones(2, 3), torch.ones(3, 2), B.Cpu)
    assert used == B.Cpu and tuple(c.shape) == (2, 2) and float(c[0, 0]) == 3.0
    _, fell_back = K.kernel_matmul_with_backend(torch.ones(2, 3), torch.ones(3, 2), B.Amd)
    assert fell_back == B.Cpu                                        # no such kernel: the CPU product, and it says so


def test_nvidia_source_names_the_blackwell_instructions():
    src = K.NVIDIA_PTX_KERNEL
    for needle in ("tcgen05", "__global__", "mbar", "tma_load", "tmem_alloc"):
        assert needle in src, needle


def test_kernel_source_for_each_backend_is_not_empty():
    for b in (B.Nvidia, B.Apple, B.Amd):
        assert K.kernel_source(b)
    assert "No kernel" in K.APPLE_MSL_KERNEL and "No kernel" in K.AMD_HIP_KERNEL


def test_extract_kernels_writes_every_source_file(tmp_path):
    paths = K.extract_kernels(str(tmp_path / "kernels"))
    assert len(paths) >= 3 and any(p.endswith("gemm_sm100.cu") for p in paths)
    for p in paths:
        assert os.path.getsize(p) > 0


def test_backend_report_is_informative():
    r = K.backend_report()
    for needle in ("Backend Report", "Tile", "Arith intensity", "ACTIVE"):
        assert needle in r, needle


def test_active_backend_is_cached():
    assert K.active_backend() is K.active_backend()


def test_set_backend_refuses_what_is_not_built():
    with pytest.raises(ValueError):
        K.set_backend(B.Apple)
    before = K.active_backend()
    K.set_backend(B.Cpu)
    assert K.active_backend() == B.Cpu
    if before != B.Cpu:
        K.set_backend(before)


def test_kernel_matmul_larger():
    torch.manual_seed(0)
    m, k, n = 64, 128, 32
    a, b = torch.randn(m, k), torch.randn(k, n)
    c, _ = K.kernel_matmul(a, b)
    assert tuple(c.shape) == (m, n) and bool(torch.isfinite(c).all())
    assert float((c.float().cpu() - a @ b).abs().max()) < 0.5       # bf16 operands on the GPU path
