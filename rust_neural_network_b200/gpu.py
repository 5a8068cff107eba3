"""GPU backend surface (rust-nn src/gpu.rs and src/gpu_kernels.rs).

The reference carries a WebGPU side path (WGSL shaders behind `GpuBackend`) and three never-launched
kernel sources (PTX / HIP / MSL) behind `GpuBackendKind`. Here the GPU is the main path, so this
module is a thin veneer: `GpuBackend` methods and the `gpu_*` helpers call the sm_100a kernels that
everything else uses (the shader arithmetic - GEMM with alpha/beta, fused linear + ReLU, softmax
attention, in-place activation - is covered by the GEMM, flash-attention and elementwise kernels),
and fall back to the CPU reference path when no CUDA device is present, as the reference's helpers
fall back to its CPU BLAS (src/gpu.rs:589-620).

`GpuBackendKind` keeps the reference's five names for API parity; only `Nvidia` (this build's
sm_100a kernels) and `Cpu` are ever active. `kernel_source` returns the CUDA source of the GEMM.
"""
from __future__ import annotations

import dataclasses
import enum
import os
import shutil
from pathlib import Path
from typing import List, Optional, Tuple

import torch

from .ops import functional as F
from .ops import gemm as G
from .ops import kernels as K

_CSRC = Path(__file__).resolve().parent.parent / "csrc"


class GpuBackendKind(enum.Enum):
    Nvidia = "NVIDIA CUDA (sm_100a, tcgen05)"
    Amd = "AMD ROCm (HIP)"
    Apple = "Apple Metal (MSL)"
    WebGpu = "WebGPU (Vulkan/DX12/Metal)"
    Cpu = "CPU (reference path)"

    def __str__(self):
        return self.value


def detect_backend() -> GpuBackendKind:
    return GpuBackendKind.Nvidia if torch.cuda.is_available() else GpuBackendKind.Cpu


@dataclasses.dataclass(frozen=True)
class TileConfig:
    """GEMM tiling of a backend: block tile bm x bn x bk, per-thread tile tm x tn, warp width."""
    bm: int
    bn: int
    bk: int
    tm: int
    tn: int
    warp_size: int
    elem_bytes: int = 4

    @staticmethod
    def b200() -> "TileConfig":
        """The tcgen05 GEMM of this build: 128 x 256 x 64 bf16 tiles, accumulator in TMEM, one row per epilogue thread."""
        return TileConfig(128, 256, 64, 1, 64, 32, 2)

    @staticmethod
    def nvidia() -> "TileConfig":
        return TileConfig.b200()

    @staticmethod
    def amd() -> "TileConfig":
        return TileConfig(128, 256, 64, 4, 4, 64)

    @staticmethod
    def apple() -> "TileConfig":
        return TileConfig(64, 64, 16, 8, 8, 32)

    @staticmethod
    def cpu() -> "TileConfig":
        return TileConfig(64, 256, 256, 1, 1, 1)

    @staticmethod
    def for_backend(backend: GpuBackendKind) -> "TileConfig":
        return {GpuBackendKind.Nvidia: TileConfig.nvidia, GpuBackendKind.Amd: TileConfig.amd, GpuBackendKind.Apple: TileConfig.apple}.get(backend, TileConfig.cpu)()

    def shared_mem_bytes(self) -> int:
        return (self.bm * self.bk + self.bk * self.bn) * self.elem_bytes

    def arithmetic_intensity(self) -> float:
        """FMAs per byte of one k-slice of a block tile."""
        return self.bm * self.bn / ((self.bm * self.bk + self.bk * self.bn) * self.elem_bytes)


_active: Optional[GpuBackendKind] = None


def active_backend() -> GpuBackendKind:
    global _active
    if _active is None:
        _active = detect_backend()
    return _active


def set_backend(backend: GpuBackendKind) -> None:
    """Selects Cpu or Nvidia; a backend this build has no kernels for is refused."""
    global _active
    if backend not in (GpuBackendKind.Nvidia, GpuBackendKind.Cpu):
        raise ValueError(f"{backend} kernels are not part of this build (sm_100a only)")
    if backend is GpuBackendKind.Nvidia and not torch.cuda.is_available():
        raise RuntimeError("no CUDA device present")
    _active = backend


def _dev(t: torch.Tensor, backend: GpuBackendKind) -> torch.Tensor:
    return t.cuda() if (backend is GpuBackendKind.Nvidia and not t.is_cuda) else t


def kernel_matmul_with_backend(a: torch.Tensor, b: torch.Tensor, backend: GpuBackendKind) -> Tuple[torch.Tensor, GpuBackendKind]:
    """[m, k] @ [k, n] on the given backend; returns (C fp32, backend that ran)."""
    if backend not in (GpuBackendKind.Nvidia, GpuBackendKind.Cpu) or (backend is GpuBackendKind.Nvidia and not torch.cuda.is_available()):
        backend = GpuBackendKind.Cpu
    a2, b2 = _dev(a.detach(), backend), _dev(b.detach(), backend)
    if backend is GpuBackendKind.Cpu:
        a2, b2 = a2.cpu(), b2.cpu()
    c = G.gemm(a2, b2, b_mn=True, out_dtype=torch.float32)
    return c.to(a.device), backend


def kernel_matmul(a: torch.Tensor, b: torch.Tensor) -> Tuple[torch.Tensor, GpuBackendKind]:
    return kernel_matmul_with_backend(a, b, active_backend())


def kernel_source(backend: GpuBackendKind) -> str:
    if backend is GpuBackendKind.Nvidia:
        src = _CSRC / "gemm" / "gemm_sm100.cu"
        if src.exists():
            return src.read_text()
        return "// gemm_sm100.cu is not shipped with this installation\n"
    return "// No kernel for this platform in this build; the CPU reference path is used.\n"


def extract_kernels(out_dir: str) -> List[str]:
    """Copies every CUDA source of the build into `out_dir`; returns the written paths."""
    os.makedirs(out_dir, exist_ok=True)
    written = []
    for src in sorted(_CSRC.rglob("*.cu")) + sorted(_CSRC.rglob("*.cuh")):
        dst = os.path.join(out_dir, src.name)
        shutil.copyfile(src, dst)
        written.append(dst)
    return written


def backend_report() -> str:
    active = active_backend()
    out = "=== rust-nn (B200) GPU Kernel Backend Report ===\n\n"
    for b in GpuBackendKind:
        c = TileConfig.for_backend(b)
        out += (f"  {b} {'[ACTIVE]' if b is active else ''}\n    Tile: BM={c.bm} BN={c.bn} BK={c.bk}\n"
                f"    Shared mem: {c.shared_mem_bytes() / 1024:.1f} KB\n    Arith intensity: {c.arithmetic_intensity():.1f} FMA/byte\n"
                f"    Warp size: {c.warp_size}\n\n")
    if torch.cuda.is_available():
        p = torch.cuda.get_device_properties(torch.cuda.current_device())
        out += f"  Device: {p.name}, {p.multi_processor_count} SMs, {p.total_memory / 2 ** 30:.0f} GiB\n"
    return out


# ------------------------------------------------------------------ GpuBackend and helpers
class GpuBackend:
    """Handle on the CUDA device (`GpuBackend.new()` is None without one, src/gpu.rs:183-219)."""

    def __init__(self, device: torch.device):
        self.device = device
        p = torch.cuda.get_device_properties(device)
        self.adapter_name = p.name

    @staticmethod
    def new(index: int = 0) -> Optional["GpuBackend"]:
        if not torch.cuda.is_available():
            return None
        return GpuBackend(torch.device("cuda", index))

    def _put(self, t: torch.Tensor) -> torch.Tensor:
        return t.detach().to(self.device)

    def matmul(self, a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
        return self.matmul_ab(a, b, 1.0, 0.0)

    def matmul_ab(self, a: torch.Tensor, b: torch.Tensor, alpha: float, beta: float, c: Optional[torch.Tensor] = None) -> torch.Tensor:
        """alpha * A B + beta * C (C defaults to zeros, as the shader's freshly created output buffer)."""
        r = G.gemm(self._put(a), self._put(b), b_mn=True, alpha=alpha, out_dtype=torch.float32)
        if c is not None and beta != 0.0:
            r = K.binary(r, K.unary(self._put(c).float(), "scale", beta), "add")
        return r

    def fused_linear(self, x: torch.Tensor, w: torch.Tensor, b: torch.Tensor, relu: bool) -> torch.Tensor:
        xd = self._put(x)
        return G.gemm(xd.reshape(-1, xd.shape[-1]), self._put(w).to(xd.dtype), bias=self._put(b).float(), act="relu" if relu else "none",
                      out_dtype=torch.float32).reshape(*xd.shape[:-1], w.shape[0])

    def flash_attention(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float) -> torch.Tensor:
        """Non-causal softmax(q k^T scale) v for [seq, d] or [batch, seq, d] inputs."""
        qd, kd, vd = (self._put(t) for t in (q, k, v))
        squeeze = qd.dim() == 2
        if squeeze:
            qd, kd, vd = qd[None], kd[None], vd[None]
        d = qd.shape[-1]
        if d > 128:      # beyond the flash kernels' head sizes: dense scores through the GEMM
            s = G.gemm(qd.to(torch.bfloat16), kd.to(torch.bfloat16), alpha=scale, out_dtype=torch.float32)
            o = G.gemm(torch.softmax(s, -1).to(torch.bfloat16), vd.to(torch.bfloat16), b_mn=True, out_dtype=torch.float32)
            return o[0] if squeeze else o
        hd = 64 if d <= 64 else 128      # zero-padding the head dimension changes neither the scores nor the kept outputs

        def prep(t):
            t = t.to(torch.bfloat16)
            if d != hd:
                t = torch.nn.functional.pad(t, (0, hd - d))
            return t.contiguous()[:, :, None, :]
        o = F.flash_attention(prep(qd), prep(kd), prep(vd), scale, False)[:, :, 0, :d].float()
        return o[0] if squeeze else o

    def activation(self, t: torch.Tensor, mode: int) -> torch.Tensor:
        """mode 0: ReLU, 1: sigmoid (the shader's two modes)."""
        return K.unary(self._put(t), "relu" if mode == 0 else "sigmoid")


_backend: Optional[GpuBackend] = None
_backend_probed = False


def gpu() -> Optional[GpuBackend]:
    global _backend, _backend_probed
    if not _backend_probed:
        _backend, _backend_probed = GpuBackend.new(), True
    return _backend


def has_gpu() -> bool:
    return gpu() is not None


def gpu_matmul(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    g = gpu()
    return g.matmul(a, b) if g is not None else G.gemm(a.detach(), b.detach(), b_mn=True, out_dtype=torch.float32)


def gpu_linear(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor, relu: bool) -> torch.Tensor:
    g = gpu()
    if g is not None:
        return g.fused_linear(x, w, b, relu)
    return G.gemm(x.detach().reshape(-1, x.shape[-1]), w.detach(), bias=b.detach().float(), act="relu" if relu else "none",
                  out_dtype=torch.float32).reshape(*x.shape[:-1], w.shape[0])


def gpu_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float) -> torch.Tensor:
    g = gpu()
    if g is not None:
        return g.flash_attention(q, k, v, scale)
    s = torch.softmax((q.float() @ k.float().transpose(-1, -2)) * scale, -1)
    return s @ v.float()


def gpu_relu(t: torch.Tensor) -> torch.Tensor:
    g = gpu()
    return g.activation(t, 0) if g is not None else torch.relu(t.detach())


def gpu_add(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    g = gpu()
    return K.binary(g._put(a), g._put(b), "add") if g is not None else a.detach() + b.detach()


def gpu_mul(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    g = gpu()
    return K.binary(g._put(a), g._put(b), "mul") if g is not None else a.detach() * b.detach()


from ._compat import install as _install  # noqa: E402

_install(globals())
