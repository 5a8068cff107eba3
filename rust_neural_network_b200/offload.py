"""Tiered tensor storage (rust-nn src/offload.rs): `MemoryTier`, `OffloadConfig`, `SsdTensor`,
`TieredTensor`, `TieredStore`, `OffloadModel`.

Three real tiers here: GPU (HBM), RAM (pinned host memory, so device pulls are single async DMA
copies) and SSD (the reference's spill files, read straight into pinned buffers by the C++
runtime). Eviction is least-recently-used, first GPU -> RAM against `gpu_budget_bytes`, then
RAM -> SSD against `ram_budget_bytes` (0 disables a budget, as in the reference). The reference has
no GPU tier (its `MemoryTier::Gpu` is never produced) and its store holds fp32 only; this one keeps
the tensor's dtype in RAM / HBM and writes fp32 spill files.
"""
from __future__ import annotations

import ctypes as C
import dataclasses
import enum
import itertools
import os
import time
from typing import Dict, Optional, Tuple

import numpy as np
import torch

from . import _native as nv
from .error import IoError

_P, _LL, _I = C.c_void_p, C.c_longlong, C.c_int
nv.register_sigs({
    "b200_ssd_write": [C.c_char_p, _P, _I, _P, _LL],
    "b200_ssd_header": [C.c_char_p, _P, _I, _P],
    "b200_ssd_read": [C.c_char_p, _P, _LL],
})


def _lib():
    lib = nv.host()
    lib.b200_ssd_write.restype = C.c_longlong
    return lib


class MemoryTier(enum.Enum):
    Gpu = "GPU"
    Ram = "RAM"
    Ssd = "SSD"

    def __str__(self):
        return self.value


@dataclasses.dataclass
class OffloadConfig:
    ram_budget_bytes: int = 2 * 1024 ** 3
    ssd_dir: str = dataclasses.field(default_factory=lambda: os.path.join(os.environ.get("HOME", "/tmp"), ".cache", "rust-nn", "ssd"))
    hot_cache_size: int = 32
    gpu_budget_bytes: int = 0            # 0: nothing is kept in HBM by the store
    device: Optional[str] = None

    def with_ram_budget_gb(self, gb: float) -> "OffloadConfig":
        self.ram_budget_bytes = int(gb * 1024 ** 3)
        return self

    def with_gpu_budget_gb(self, gb: float, device: str = "cuda") -> "OffloadConfig":
        self.gpu_budget_bytes, self.device = int(gb * 1024 ** 3), device
        return self

    def with_ssd_dir(self, d: str) -> "OffloadConfig":
        self.ssd_dir = str(d)
        return self

    def with_hot_cache(self, size: int) -> "OffloadConfig":
        self.hot_cache_size = size
        return self


_next_id = itertools.count()


def _pinned_like(shape, dtype) -> torch.Tensor:
    t = torch.empty(shape, dtype=dtype)
    if torch.cuda.is_available():
        try:
            return t.pin_memory()
        except RuntimeError:
            pass
    return t


class SsdTensor:
    """One spill file `[ndim u32][dims u64 ...][f32 data]`; removed when the object dies."""

    def __init__(self, path: str, shape, nbytes: int, dtype=torch.float32):
        self._path, self._shape, self._bytes, self.dtype = path, list(shape), nbytes, dtype

    @staticmethod
    def write(tensor: torch.Tensor, directory: str) -> "SsdTensor":
        os.makedirs(directory, exist_ok=True)
        path = os.path.join(directory, f"tensor_{os.getpid()}_{next(_next_id)}.bin")
        host = tensor.detach().to("cpu", torch.float32).contiguous()
        shape = np.asarray(host.shape, dtype=np.int64)
        n = _lib().b200_ssd_write(path.encode(), shape.ctypes.data if shape.size else None, host.dim(), host.data_ptr(), host.numel())
        if n < 0:
            raise IoError(f"cannot write {path}: errno {-n}")
        return SsdTensor(path, host.shape, int(n), tensor.dtype)

    def load(self) -> torch.Tensor:
        lib = _lib()
        shape = np.zeros(64, dtype=np.int64)
        numel = C.c_longlong(0)
        nd = lib.b200_ssd_header(self._path.encode(), shape.ctypes.data, 64, C.byref(numel))
        if nd < 0:
            raise IoError(f"{self._path}: file too short or unreadable")
        out = _pinned_like([int(s) for s in shape[:nd]], torch.float32)
        if lib.b200_ssd_read(self._path.encode(), out.data_ptr(), numel.value) != 0:
            raise IoError(f"{self._path}: short read")
        return out if self.dtype == torch.float32 else out.to(self.dtype)

    def evict(self) -> None:
        os.remove(self._path)

    def size_bytes(self) -> int:
        return self._bytes

    def shape(self):
        return list(self._shape)

    def path(self) -> str:
        return self._path

    def __del__(self):
        try:
            os.remove(self._path)
        except OSError:
            pass


class TieredTensor:
    def __init__(self, tensor: torch.Tensor):
        self.gpu: Optional[torch.Tensor] = tensor if tensor.is_cuda else None
        self.ram: Optional[torch.Tensor] = None if tensor.is_cuda else tensor
        self.ssd: Optional[SsdTensor] = None
        self._tier = MemoryTier.Gpu if tensor.is_cuda else MemoryTier.Ram
        self.last_access = time.monotonic()
        self._nbytes = tensor.numel() * tensor.element_size()

    @staticmethod
    def from_tensor(tensor: torch.Tensor) -> "TieredTensor":
        return TieredTensor(tensor)

    def tier(self) -> MemoryTier:
        return self._tier

    def size_bytes(self) -> int:
        return self.ssd.size_bytes() if self._tier == MemoryTier.Ssd and self.ssd is not None else self._nbytes

    def age(self) -> float:
        return time.monotonic() - self.last_access

    def demote_to_ram(self) -> None:
        if self._tier != MemoryTier.Gpu:
            return
        host = _pinned_like(self.gpu.shape, self.gpu.dtype)
        host.copy_(self.gpu, non_blocking=True)
        torch.cuda.current_stream(self.gpu.device).synchronize()
        self.ram, self.gpu, self._tier = host, None, MemoryTier.Ram

    def offload_to_ssd(self, directory: str) -> None:
        if self._tier == MemoryTier.Ssd:
            return
        src = self.gpu if self._tier == MemoryTier.Gpu else self.ram
        self.ssd = SsdTensor.write(src, directory)
        self.ram = self.gpu = None
        self._tier = MemoryTier.Ssd

    def load_to_ram(self) -> None:
        if self._tier != MemoryTier.Ssd:
            return
        self.ram = self.ssd.load()
        self.ssd = None
        self._tier = MemoryTier.Ram
        self.last_access = time.monotonic()

    def promote_to_gpu(self, device) -> None:
        if self._tier == MemoryTier.Gpu:
            return
        self.load_to_ram()
        self.gpu = self.ram.to(device, non_blocking=True)
        self.ram = None
        self._tier = MemoryTier.Gpu

    def get(self) -> torch.Tensor:
        if self._tier == MemoryTier.Ssd:
            self.load_to_ram()
        self.last_access = time.monotonic()
        return self.gpu if self._tier == MemoryTier.Gpu else self.ram


class TieredStore:
    def __init__(self, config: Optional[OffloadConfig] = None):
        self.config = config or OffloadConfig()
        try:
            os.makedirs(self.config.ssd_dir, exist_ok=True)
        except OSError:
            pass
        self.tensors: Dict[str, TieredTensor] = {}
        self._ram_usage = 0
        self._gpu_usage = 0

    @staticmethod
    def new(config: OffloadConfig) -> "TieredStore":
        return TieredStore(config)

    def _account(self, t: TieredTensor, sign: int) -> None:
        if t.tier() == MemoryTier.Ram:
            self._ram_usage += sign * t.size_bytes()
        elif t.tier() == MemoryTier.Gpu:
            self._gpu_usage += sign * t.size_bytes()

    def insert(self, name: str, tensor: torch.Tensor) -> None:
        old = self.tensors.pop(name, None)
        if old is not None:
            self._account(old, -1)
        t = TieredTensor(tensor.detach())
        self.tensors[name] = t
        self._account(t, +1)
        self.maybe_evict()

    def get(self, name: str, device=None) -> Optional[torch.Tensor]:
        """The tensor (loaded from SSD if needed; moved into HBM when `device` is a CUDA device and the
        GPU budget allows it), or None for an unknown name."""
        t = self.tensors.get(name)
        if t is None:
            return None
        self._account(t, -1)
        try:
            t.get()
            want_gpu = device is not None and torch.device(device).type == "cuda"
            if want_gpu and self.config.gpu_budget_bytes > 0:
                t.promote_to_gpu(device)
        finally:
            self._account(t, +1)
        out = t.get()
        self.maybe_evict(protect=name)
        if device is not None and out.device != torch.device(device):
            return out.to(device, non_blocking=True)
        return out

    def offload(self, name: str) -> None:
        t = self.tensors.get(name)
        if t is None:
            return
        self._account(t, -1)
        try:
            t.offload_to_ssd(self.config.ssd_dir)
        finally:
            self._account(t, +1)

    def offload_all(self) -> None:
        for name in list(self.tensors):
            self.offload(name)

    def load_all(self) -> None:
        for t in self.tensors.values():
            if t.tier() == MemoryTier.Ssd:
                t.load_to_ram()
                self._account(t, +1)

    def _coldest(self, tier: MemoryTier, protect: Optional[str]) -> Optional[str]:
        best, best_age = None, -1.0
        for name, t in self.tensors.items():
            if t.tier() == tier and name != protect and t.age() > best_age:
                best, best_age = name, t.age()
        return best

    def maybe_evict(self, protect: Optional[str] = None) -> None:
        cfg = self.config
        while cfg.gpu_budget_bytes > 0 and self._gpu_usage > cfg.gpu_budget_bytes:
            name = self._coldest(MemoryTier.Gpu, protect)
            if name is None:
                break
            t = self.tensors[name]
            self._account(t, -1)
            t.demote_to_ram()
            self._account(t, +1)
        while cfg.ram_budget_bytes > 0 and self._ram_usage > cfg.ram_budget_bytes:
            name = self._coldest(MemoryTier.Ram, protect)
            if name is None:
                break
            try:
                self.offload(name)
            except IoError:
                break

    def ram_usage(self) -> int:
        return self._ram_usage

    def gpu_usage(self) -> int:
        return self._gpu_usage

    def tier_counts(self) -> Tuple[int, int]:
        """(tensors in RAM or HBM, tensors on SSD)."""
        ssd = sum(1 for t in self.tensors.values() if t.tier() == MemoryTier.Ssd)
        return len(self.tensors) - ssd, ssd

    def ssd_usage(self) -> int:
        return sum(t.size_bytes() for t in self.tensors.values() if t.tier() == MemoryTier.Ssd)

    def __repr__(self):
        return (f"TieredStore {{ ram_usage_mb: {self._ram_usage // 1024 // 1024}, ram_budget_mb: "
                f"{self.config.ram_budget_bytes // 1024 // 1024}, num_tensors: {len(self.tensors)} }}")


class OffloadModel:
    """Wraps a model whose parameters live in a `TieredStore`; `offload()` spills them to SSD and
    releases their memory, `forward` brings them back first (src/offload.rs:480-540)."""

    def __init__(self, model, config: Optional[OffloadConfig] = None):
        self.model = model
        self.store = TieredStore(config)
        self._params = list(model.parameters())
        for i, p in enumerate(self._params):
            self.store.insert(f"param_{i}", p.data)
        self.offloaded = False

    def offload(self) -> None:
        self.store.offload_all()
        for p in self._params:                     # drop the live copies: the spill files are now the only ones
            p.data = torch.empty(0, dtype=p.dtype, device=p.device)
            if hasattr(p, "_lp"):
                p._lp = None
        self.offloaded = True

    def load(self) -> None:
        for i, p in enumerate(self._params):
            dev = p.device
            t = self.store.get(f"param_{i}")
            p.data = t.to(dev) if t.device != dev else t
            if hasattr(p, "_lp_version"):
                p._lp_version = -1
        self.offloaded = False

    def forward(self, x):
        if self.offloaded:
            self.load()
        return self.model(x)

    __call__ = forward

    def ram_usage(self) -> int:
        return self.store.ram_usage()

    def ssd_usage(self) -> int:
        return self.store.ssd_usage()

    def memory_report(self) -> str:
        ram, ssd = self.store.tier_counts()
        return (f"OffloadModel memory: {ram + ssd} tensors (RAM: {ram}, SSD: {ssd}), RAM: {self.ram_usage() / 1024 / 1024:.1f} MB, "
                f"SSD: {self.ssd_usage() / 1024 / 1024:.1f} MB")


from ._compat import install as _install  # noqa: E402

_install(globals())
