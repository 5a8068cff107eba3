// Allocation-free entry point of the optimizer library.
//
// This entry point has no counterpart in the reference (rust-nn has no device code at all); it
// exists for callers of THIS library that cannot allocate device memory at the point of the call:
// code running while the device allocator is off limits (a frozen memory pool, a step that is being
// captured or replayed, a latency-critical section that must not enter the driver's allocator) and
// host programs that receive device pointers from another runtime and own no allocator. Such a
// caller passes only its inputs and outputs; the per-segment scratch that b200_muon_rms asks its
// caller for is a fixed array inside the library instead.
//
// Limits and rules:
//   * nseg <= B200_NOALLOC_MAX_SEGMENTS, otherwise the call returns B200_NOALLOC_TOO_MANY_SEGMENTS and
//     launches nothing;
//   * the library keeps B200_NOALLOC_MAX_SEGMENTS * 4 bytes per GPU for the life of the process;
//   * the first call on each device resolves the array's device address and should be made before
//     any stream capture begins; the address is cached per device ordinal without a lock (two threads
//     racing on a device's first call both look up, and store, the same value);
//   * the array is shared by all calls and is cleared on the caller's stream at the start of each
//     call; calls that may overlap on the GPU must be ordered by the caller.
#pragma once
#include <cuda_runtime.h>

#define B200_NOALLOC_MAX_SEGMENTS 4096

enum {
  B200_NOALLOC_TOO_MANY_SEGMENTS = -10,
  B200_NOALLOC_BAD_DEVICE = -11,
  B200_NOALLOC_SYMBOL_LOOKUP_FAILED = -12,
};

// Muon (per-tensor RMS-normalised gradient, then momentum SGD) over flat fp32 buffers, exactly as
// b200_muon_rms, without caller-provided scratch.
//   p, g, buf   : flat fp32 parameter / gradient / momentum buffers (device)
//   shadow_bf16 : optional flat bf16 copy of the parameters, rewritten by the same kernel (or null)
//   seg_off     : device array of nseg [begin, end) element ranges (int64 pairs)
// Returns 0 on success, one of the codes above, or a CUDA error code from the launch.
#ifdef __cplusplus
extern "C" {
#endif
int b200_muon_rms_noalloc(float* p, const float* g, float* buf, void* shadow_bf16, const long long* seg_off,
                          int nseg, float lr, float momentum, float eps, cudaStream_t st);
#ifdef __cplusplus
}
#endif
