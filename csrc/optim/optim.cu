// O1: fused optimizers over flat fp32 master buffers (one launch for every parameter of a model),
// with the bf16 shadow copy of the weights written by the same kernel.
//   Adam   : m = b1 m + (1-b1) g ; v = b2 v + (1-b2) g^2 ; p -= lr_t * m / (sqrt(v) * c2 + eps)
//            reference form (rust-nn src/optim.rs:91-111,170-212): lr_t = lr*sqrt(1-b2^t)/(1-b1^t), c2 = 1;
//            torch form: lr_t = lr/(1-b1^t), c2 = 1/sqrt(1-b2^t).
//   SGD    : buf = g on the first step, else momentum*buf + g ; p -= lr * buf   (src/optim.rs:29-47)
//   RMSprop: v = a v + (1-a) g^2 ; p -= lr * g / (sqrt(v) + eps)                 (src/optim.rs:246-256)
//   Muon (reference variant, src/optim.rs:284-307): g is divided by its per-tensor RMS, then momentum SGD.
// The step counter lives on the device so that a captured CUDA graph replays correctly.
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cstdint>

namespace b200 {

struct AdamHyper { float lr, b1, b2, eps, weight_decay; int torch_form; };

__global__ void adam_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m,
                            float* __restrict__ v, __nv_bfloat16* __restrict__ shadow, long long n, AdamHyper h,
                            const float* __restrict__ step_ptr, const float* __restrict__ grad_scale_ptr) {
  const float t = *step_ptr + 1.f;
  const float bc1 = 1.f - powf(h.b1, t), bc2 = 1.f - powf(h.b2, t);
  const float lr_t = h.torch_form ? h.lr / bc1 : h.lr * sqrtf(bc2) / bc1;
  const float c2 = h.torch_form ? rsqrtf(bc2) : 1.f;
  const float gs = grad_scale_ptr ? *grad_scale_ptr : 1.f;
  const float ob1 = 1.f - h.b1, ob2 = 1.f - h.b2;
  long long i = (blockIdx.x * (long long)blockDim.x + threadIdx.x) * 4;
  const long long stride = (long long)gridDim.x * blockDim.x * 4;
  for (; i + 3 < n; i += stride) {
    // every byte is touched once per step: streaming loads / stores keep the 4 read and 4 write streams from evicting
    // one another (and the bf16 shadow, which the next forward reads) out of L2
    float4 pp = __ldcs(reinterpret_cast<const float4*>(p + i)), gg = __ldcs(reinterpret_cast<const float4*>(g + i));
    float4 mm = __ldcs(reinterpret_cast<const float4*>(m + i)), vv = __ldcs(reinterpret_cast<const float4*>(v + i));
    float* P = &pp.x; float* G = &gg.x; float* M = &mm.x; float* V = &vv.x;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float gr = G[j] * gs;
      if (h.weight_decay != 0.f) P[j] -= h.lr * h.weight_decay * P[j];
      M[j] = h.b1 * M[j] + ob1 * gr;
      V[j] = h.b2 * V[j] + ob2 * gr * gr;
      P[j] -= lr_t * M[j] / (sqrtf(V[j]) * c2 + h.eps);
    }
    __stcs(reinterpret_cast<float4*>(p + i), pp); __stcs(reinterpret_cast<float4*>(m + i), mm); __stcs(reinterpret_cast<float4*>(v + i), vv);
    if (shadow) {
      __nv_bfloat162 a = __floats2bfloat162_rn(pp.x, pp.y), b = __floats2bfloat162_rn(pp.z, pp.w);
      uint2 o; o.x = *reinterpret_cast<uint32_t*>(&a); o.y = *reinterpret_cast<uint32_t*>(&b);
      *reinterpret_cast<uint2*>(shadow + i) = o;
    }
  }
  // tail (n not a multiple of 4): handled by the first threads
  long long tail0 = n & ~3ll;
  long long k = tail0 + blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (k < n) {
    float gr = g[k] * gs, pk = p[k];
    if (h.weight_decay != 0.f) pk -= h.lr * h.weight_decay * pk;
    float mk = h.b1 * m[k] + ob1 * gr, vk = h.b2 * v[k] + ob2 * gr * gr;
    pk -= lr_t * mk / (sqrtf(vk) * c2 + h.eps);
    p[k] = pk; m[k] = mk; v[k] = vk;
    if (shadow) shadow[k] = __float2bfloat16(pk);
  }
}

__global__ void sgd_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ buf,
                           __nv_bfloat16* __restrict__ shadow, long long n, float lr, float momentum,
                           const float* __restrict__ step_ptr, const float* __restrict__ grad_scale_ptr) {
  const bool first = (*step_ptr == 0.f);
  const float gs = grad_scale_ptr ? *grad_scale_ptr : 1.f;
  long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (; i < n; i += stride) {
    float gr = g[i] * gs, pk = p[i];
    if (buf && momentum != 0.f) { float b = first ? gr : momentum * buf[i] + gr; buf[i] = b; gr = b; }
    pk -= lr * gr; p[i] = pk;
    if (shadow) shadow[i] = __float2bfloat16(pk);
  }
}

__global__ void rmsprop_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ v,
                               __nv_bfloat16* __restrict__ shadow, long long n, float lr, float alpha, float eps,
                               const float* __restrict__ grad_scale_ptr) {
  const float gs = grad_scale_ptr ? *grad_scale_ptr : 1.f;
  long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (; i < n; i += stride) {
    float gr = g[i] * gs;
    float vk = alpha * v[i] + (1.f - alpha) * gr * gr; v[i] = vk;
    float pk = p[i] - lr * gr / (sqrtf(vk) + eps); p[i] = pk;
    if (shadow) shadow[i] = __float2bfloat16(pk);
  }
}

// Muon, reference variant: per-tensor RMS normalisation then momentum SGD. One block per segment
// slice; seg_sumsq[s] holds sum(g^2) of segment s (computed by muon_sumsq_kernel).
__global__ void muon_sumsq_kernel(const float* __restrict__ g, const long long* __restrict__ seg_off, int nseg,
                                  float* __restrict__ seg_sumsq) {
  int s = blockIdx.y;
  long long a = seg_off[2 * s], b = seg_off[2 * s + 1];
  float acc = 0.f;
  for (long long i = a + blockIdx.x * (long long)blockDim.x + threadIdx.x; i < b; i += (long long)gridDim.x * blockDim.x)
    acc += g[i] * g[i];
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  __shared__ float sh[32];
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    acc = threadIdx.x < (blockDim.x >> 5) ? sh[threadIdx.x] : 0.f;
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (threadIdx.x == 0) atomicAdd(seg_sumsq + s, acc);
  }
}
__global__ void muon_rms_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ buf,
                                __nv_bfloat16* __restrict__ shadow, const long long* __restrict__ seg_off, int nseg,
                                const float* __restrict__ seg_sumsq, float lr, float momentum, float eps) {
  int s = blockIdx.y;
  long long a = seg_off[2 * s], b = seg_off[2 * s + 1];
  float rms = fmaxf(sqrtf(seg_sumsq[s] / (float)(b - a > 0 ? b - a : 1)), eps);
  for (long long i = a + blockIdx.x * (long long)blockDim.x + threadIdx.x; i < b; i += (long long)gridDim.x * blockDim.x) {
    float gn = g[i] / rms;
    float bb = momentum * buf[i] + gn; buf[i] = bb;
    float pk = p[i] - lr * bb; p[i] = pk;
    if (shadow) shadow[i] = __float2bfloat16(pk);
  }
}

// scalars[0] = sum of squares of all grads (input) -> scalars[1] = clip coefficient min(1, max_norm/(norm+1e-6))
__global__ void clip_coef_kernel(float* scalars, float max_norm) {
  float norm = sqrtf(scalars[0]);
  scalars[1] = fminf(1.f, max_norm / (norm + 1e-6f));
  scalars[2] = norm;
}
__global__ void incr_kernel(float* step) { *step += 1.f; }

}  // namespace b200

using namespace b200;

static inline int ogrid(long long n, int per_thread) {
  long long g = (n / per_thread + 255) / 256; if (g < 1) g = 1; if (g > 148 * 8) g = 148 * 8; return (int)g;
}

extern "C" {

int b200_adam(float* p, const float* g, float* m, float* v, void* shadow_bf16, long long n, float lr, float b1,
              float b2, float eps, float weight_decay, int torch_form, const float* step_ptr,
              const float* grad_scale_ptr, cudaStream_t st) {
  if (n <= 0) return 0;
  AdamHyper h{lr, b1, b2, eps, weight_decay, torch_form};
  adam_kernel<<<ogrid(n, 4), 256, 0, st>>>(p, g, m, v, (__nv_bfloat16*)shadow_bf16, n, h, step_ptr, grad_scale_ptr);
  return (int)cudaGetLastError();
}
int b200_sgd(float* p, const float* g, float* buf, void* shadow_bf16, long long n, float lr, float momentum,
             const float* step_ptr, const float* grad_scale_ptr, cudaStream_t st) {
  if (n <= 0) return 0;
  sgd_kernel<<<ogrid(n, 1), 256, 0, st>>>(p, g, buf, (__nv_bfloat16*)shadow_bf16, n, lr, momentum, step_ptr, grad_scale_ptr);
  return (int)cudaGetLastError();
}
int b200_rmsprop(float* p, const float* g, float* v, void* shadow_bf16, long long n, float lr, float alpha, float eps,
                 const float* grad_scale_ptr, cudaStream_t st) {
  if (n <= 0) return 0;
  rmsprop_kernel<<<ogrid(n, 1), 256, 0, st>>>(p, g, v, (__nv_bfloat16*)shadow_bf16, n, lr, alpha, eps, grad_scale_ptr);
  return (int)cudaGetLastError();
}
// seg_off: device array of nseg [begin, end) pairs into the flat buffers; seg_sumsq: device scratch of nseg floats
int b200_muon_rms(float* p, const float* g, float* buf, void* shadow_bf16, const long long* seg_off, int nseg,
                  float* seg_sumsq, float lr, float momentum, float eps, cudaStream_t st) {
  if (nseg <= 0) return 0;
  cudaMemsetAsync(seg_sumsq, 0, sizeof(float) * nseg, st);
  dim3 grid(32, nseg);
  muon_sumsq_kernel<<<grid, 256, 0, st>>>(g, seg_off, nseg, seg_sumsq);
  muon_rms_kernel<<<grid, 256, 0, st>>>(p, g, buf, (__nv_bfloat16*)shadow_bf16, seg_off, nseg, seg_sumsq, lr, momentum, eps);
  return (int)cudaGetLastError();
}
int b200_clip_coef(float* scalars, float max_norm, cudaStream_t st) {
  clip_coef_kernel<<<1, 1, 0, st>>>(scalars, max_norm);
  return (int)cudaGetLastError();
}
int b200_incr_step(float* step, cudaStream_t st) {
  incr_kernel<<<1, 1, 0, st>>>(step);
  return (int)cudaGetLastError();
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------
// Allocation-free variant of b200_muon_rms (declared in optim_noalloc.h).
//
// b200_muon_rms needs one float of scratch per parameter segment (the per-tensor sum of squared
// gradients) and takes that scratch from its caller. Some callers have no way to provide it: code
// that runs where the device allocator must not be touched - inside a region that a framework has
// frozen (a captured or replayed stream, a memory pool that is closed for the duration of a step), in
// a signal-safe or real-time section, or in a host program that was handed device pointers by
// another runtime and owns no allocator of its own. For them the scratch lives in a fixed array
// inside this library: every GPU that loads the library holds B200_NOALLOC_MAX_SEGMENTS floats
// (16 KiB) until the process exits, and this entry point calls no cudaMalloc / cudaFree and no
// allocating library routine.
//
// Contract:
//   * at most B200_NOALLOC_MAX_SEGMENTS segments; more is rejected with B200_NOALLOC_TOO_MANY_SEGMENTS
//     (and a message on stderr) before anything is launched;
//   * the first call on a device looks up the device address of the array (cudaGetSymbolAddress, with
//     that device current) and remembers it; make that first call outside any stream capture;
//   * all calls share the one array, which keeps the previous call's sums: the entry point clears
//     the part it uses on the caller's stream before accumulating into it, and two calls that
//     overlap on the GPU (different streams, no ordering between them) race on it - serialise them.
#include "optim_noalloc.h"
#include <cstdio>

namespace b200 {

static __device__ __align__(256) float g_noalloc_seg_sumsq[B200_NOALLOC_MAX_SEGMENTS];

constexpr int NOALLOC_MAX_DEVICES = 64;
// Device address of g_noalloc_seg_sumsq per device ordinal. In host code the array's NAME is only a
// stand-in for the symbol, not a device address, so it must never be passed to a kernel directly.
static float* g_noalloc_scratch_ptr[NOALLOC_MAX_DEVICES] = {nullptr};

}  // namespace b200

extern "C" int b200_muon_rms_noalloc(float* p, const float* g, float* buf, void* shadow_bf16, const long long* seg_off,
                                     int nseg, float lr, float momentum, float eps, cudaStream_t st) {
  using namespace b200;
  if (nseg <= 0) return 0;
  if (nseg > B200_NOALLOC_MAX_SEGMENTS) {
    fprintf(stderr, "b200_muon_rms_noalloc: %d segments exceed the built-in scratch of %d segments; "
                    "use b200_muon_rms with caller-provided scratch\n", nseg, B200_NOALLOC_MAX_SEGMENTS);
    return B200_NOALLOC_TOO_MANY_SEGMENTS;
  }
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= NOALLOC_MAX_DEVICES) return B200_NOALLOC_BAD_DEVICE;
  float* scratch = g_noalloc_scratch_ptr[dev];
  if (scratch == nullptr) {
    // one-time set-up for this device (it is the current device here)
    void* sym = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&sym, g_noalloc_seg_sumsq);
    if (e != cudaSuccess || sym == nullptr) {
      fprintf(stderr, "b200_muon_rms_noalloc: cudaGetSymbolAddress failed: %s\n", cudaGetErrorString(e));
      return B200_NOALLOC_SYMBOL_LOOKUP_FAILED;
    }
    scratch = static_cast<float*>(sym);
    g_noalloc_scratch_ptr[dev] = scratch;
  }
  // the array still holds the sums of the previous call: clear the part this call accumulates into
  if (cudaMemsetAsync(scratch, 0, sizeof(float) * nseg, st) != cudaSuccess) return (int)cudaGetLastError();
  dim3 grid(32, nseg);
  muon_sumsq_kernel<<<grid, 256, 0, st>>>(g, seg_off, nseg, scratch);
  muon_rms_kernel<<<grid, 256, 0, st>>>(p, g, buf, (__nv_bfloat16*)shadow_bf16, seg_off, nseg, scratch, lr, momentum, eps);
  return (int)cudaGetLastError();
}
