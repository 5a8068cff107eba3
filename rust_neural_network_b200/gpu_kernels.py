"""Kernel-selection surface of the reference (rust-nn src/gpu_kernels.rs), re-exported from `gpu`."""
from .gpu import (GpuBackendKind, TileConfig, active_backend, backend_report, detect_backend, extract_kernels, kernel_matmul,  # noqa: F401
                  kernel_matmul_with_backend, kernel_source, set_backend)
from .gpu import GpuBackendKind as _K, kernel_source as _src

NVIDIA_PTX_KERNEL = _src(_K.Nvidia)          # the CUDA source of the sm_100a GEMM
AMD_HIP_KERNEL = _src(_K.Amd)                # no such kernel in this build: a one-line comment
APPLE_MSL_KERNEL = _src(_K.Apple)



from ._compat import install as _install  # noqa: E402

_install(globals(), imported=True)
