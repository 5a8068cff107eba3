// Programmatic dependent launch (PDL). A kernel launched through `launch_pdl` may start while its predecessor on the
// stream is still running: its blocks are dispatched as soon as every block of the predecessor has executed
// `pdl_trigger()` (or exited), they run their prologue (barrier set-up, tensor-memory allocation, descriptor prefetch)
// and then block in `pdl_wait()` until the predecessor has completed and its writes are visible. What is saved is the
// launch latency and the prologue of every kernel - about a third of the time of the 8-40 us kernels a small per-GPU
// batch is made of. The rules every kernel launched this way follows:
//   * `pdl_trigger()` first thing, so that the next kernel can be dispatched early;
//   * `pdl_wait()` before the first access to global memory (read OR write);
// a kernel that is launched WITHOUT the attribute runs both instructions as no-ops, and a kernel without them that
// follows on the stream is ordered after the full completion of everything before it, as usual. Inside a stream capture
// the launches become programmatic dependency edges of the CUDA graph. `b200_set_pdl(0)` turns the attribute off.
#pragma once
#include <cuda_runtime.h>
#include <utility>

namespace b200 {

inline int g_pdl_enabled = 1;

__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = g_pdl_enabled ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

// the same, as clusters of two CTAs along x (grid.x must be even)
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl_cluster2(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = g_pdl_enabled ? 2 : 1;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

}  // namespace b200
