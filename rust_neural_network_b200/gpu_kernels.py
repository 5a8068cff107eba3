"""Kernel-selection surface of the reference (rust-nn src/gpu_kernels.rs), re-exported from `gpu`."""
from .gpu import (GpuBackendKind, TileConfig, active_backend, backend_report, detect_backend, extract_kernels, kernel_matmul,  # noqa: F401
                  kernel_matmul_with_backend, kernel_source, set_backend)
