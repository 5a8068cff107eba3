// L1: fused softmax cross-entropy (forward value and logits gradient in one launch) for integer
// labels (LM head, vocab 32000) and for dense one-hot / soft targets, and
// L2: the elementwise losses (MSE, L1, Huber, BCE, BCE-with-logits) with their gradients.
// Math restates rust-nn src/tensor.rs:464-606 (forward) and 1379-1467 (backward):
// cross-entropy is the mean over the batch of -sum_c t_c log softmax(x)_c with gradient
// (softmax(x) * sum(t) - t) / batch; BCE clamps probabilities to [1e-12, 1-1e-12].
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cstdint>
#include <cmath>

namespace b200 {

template <typename T> __device__ __forceinline__ float lf(const T* p);
template <> __device__ __forceinline__ float lf<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float lf<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void sf(T* p, float v);
template <> __device__ __forceinline__ void sf<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void sf<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16(v); }

template <typename T, int N> struct alignas(sizeof(T) * N) PackL { T v[N]; };

__device__ __forceinline__ float ex2f(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ void online_combine(float& m, float& s, float m2, float s2) {
  float nm = fmaxf(m, m2);
  if (nm == -INFINITY) { s = 0.f; m = nm; return; }
  s = s * __expf(m - nm) + s2 * __expf(m2 - nm);
  m = nm;
}

// One block per row. Pass 1: online (max, sum-exp) with 16-byte loads. Pass 2 (L2-resident re-read):
// write (softmax - onehot) * grad_scale. Per-row loss goes to loss_rows; the mean is accumulated
// into loss_sum with one atomic per row. Labels < 0 (ignore) contribute nothing.
template <typename T>
__global__ void __launch_bounds__(512, 3) ce_label_kernel(const T* __restrict__ logits, const long long* __restrict__ labels,
                                T* __restrict__ dlogits, float* __restrict__ loss_rows, float* __restrict__ loss_sum,
                                int V, long long ld, float grad_scale, float loss_scale) {
  constexpr int N = 16 / sizeof(T);
  using P = PackL<T, N>;
  const long long row = blockIdx.x;
  const T* xr = logits + row * ld;
  const long long label = labels[row];
  // read before any gradient is written: dlogits may alias logits (in-place use by the fused LM head)
  const float x_label = (threadIdx.x == 0 && label >= 0 && label < V) ? lf(xr + label) : 0.f;
  float m = -INFINITY, s = 0.f;
  const bool vec = (ld % N == 0) && ((reinterpret_cast<uintptr_t>(logits) & 15) == 0);
  const int nv = vec ? V / N : 0;
  int i = threadIdx.x;
  // four packets per thread in flight: with one, a 512-thread block keeps 8 KB outstanding and the pass runs at ~4 TB/s
  for (; i + 3 * (int)blockDim.x < nv; i += 4 * blockDim.x) {
    P p[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) p[u] = reinterpret_cast<const P*>(xr)[i + u * blockDim.x];
    float lm = -INFINITY;
#pragma unroll
    for (int u = 0; u < 4; ++u)
#pragma unroll
      for (int j = 0; j < N; ++j) lm = fmaxf(lm, lf(&p[u].v[j]));
    float ls = 0.f;
    const float nl = -lm * kLog2e;
#pragma unroll
    for (int u = 0; u < 4; ++u)
#pragma unroll
      for (int j = 0; j < N; ++j) ls += ex2f(fmaf(lf(&p[u].v[j]), kLog2e, nl));
    online_combine(m, s, lm, ls);
  }
  for (; i < nv; i += blockDim.x) {
    P p = reinterpret_cast<const P*>(xr)[i];
    float lm = -INFINITY;
#pragma unroll
    for (int j = 0; j < N; ++j) lm = fmaxf(lm, lf(&p.v[j]));
    float ls = 0.f;
#pragma unroll
    for (int j = 0; j < N; ++j) ls += __expf(lf(&p.v[j]) - lm);
    online_combine(m, s, lm, ls);
  }
  for (int c = nv * N + threadIdx.x; c < V; c += blockDim.x) online_combine(m, s, lf(xr + c), 1.f);
  __shared__ float sm[32], ss[32];
  for (int o = 16; o > 0; o >>= 1) {
    float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, s, o);
    online_combine(m, s, m2, s2);
  }
  if ((threadIdx.x & 31) == 0) { sm[threadIdx.x >> 5] = m; ss[threadIdx.x >> 5] = s; }
  __syncthreads();
  if (threadIdx.x < 32) {
    int nw = blockDim.x >> 5;
    m = threadIdx.x < nw ? sm[threadIdx.x] : -INFINITY;
    s = threadIdx.x < nw ? ss[threadIdx.x] : 0.f;
    for (int o = 16; o > 0; o >>= 1) {
      float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, s, o);
      online_combine(m, s, m2, s2);
    }
    if (threadIdx.x == 0) { sm[0] = m; ss[0] = s; }
  }
  __syncthreads();
  m = sm[0]; s = ss[0];
  const float lse = m + logf(s);
  const bool valid = label >= 0 && label < V;
  if (threadIdx.x == 0) {
    float l = valid ? lse - x_label : 0.f;
    if (loss_rows) loss_rows[row] = l;
    if (loss_sum && valid) atomicAdd(loss_sum, l * loss_scale);
  }
  if (!dlogits) return;
  T* dr = dlogits + row * ld;
  const float gs = valid ? grad_scale : 0.f;
  // softmax * gs as one exponential: 2^(x log2e - (m log2e + log2 s - log2 gs)); an ignored row (gs = 0) gets 2^-inf = 0.
  // The label's element is rewritten by thread 0 after the row is out (it kept x[label] from before the first write).
  const float c2 = valid ? m * kLog2e + log2f(s) - log2f(grad_scale) : INFINITY;
  auto grad_packet = [&](const P& p, int idx) {
    P o;
#pragma unroll
    for (int j = 0; j < N; ++j) sf(&o.v[j], ex2f(fmaf(lf(&p.v[j]), kLog2e, -c2)));
    reinterpret_cast<P*>(dr)[idx] = o;
  };
  i = threadIdx.x;
  for (; i + (int)blockDim.x < nv; i += 2 * blockDim.x) {            // the re-read hits L2; two packets in flight per thread
    const P p0 = reinterpret_cast<const P*>(xr)[i], p1 = reinterpret_cast<const P*>(xr)[i + blockDim.x];
    grad_packet(p0, i);
    grad_packet(p1, i + blockDim.x);
  }
  for (; i < nv; i += blockDim.x) grad_packet(reinterpret_cast<const P*>(xr)[i], i);
  for (int c = nv * N + threadIdx.x; c < V; c += blockDim.x) sf(dr + c, ex2f(fmaf(lf(xr + c), kLog2e, -c2)));
  __syncthreads();
  if (threadIdx.x == 0 && valid) sf(dr + label, ex2f(fmaf(x_label, kLog2e, -c2)) - gs);
}

// dense targets (one-hot or soft): loss_row = -sum_c t_c * log(max(softmax_c, 1e-12)); grad = (p*sum(t) - t)*scale
template <typename T>
__global__ void ce_dense_kernel(const T* __restrict__ logits, const T* __restrict__ target, T* __restrict__ dlogits,
                                float* __restrict__ loss_sum, int V, float grad_scale, float loss_scale) {
  const long long row = blockIdx.x;
  const T* xr = logits + row * (long long)V; const T* tr = target + row * (long long)V;
  float m = -INFINITY, s = 0.f, tsum = 0.f;
  for (int c = threadIdx.x; c < V; c += blockDim.x) { online_combine(m, s, lf(xr + c), 1.f); tsum += lf(tr + c); }
  __shared__ float sm[32], ss[32], st[32];
  for (int o = 16; o > 0; o >>= 1) {
    float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, s, o);
    online_combine(m, s, m2, s2);
    tsum += __shfl_xor_sync(0xffffffffu, tsum, o);
  }
  if ((threadIdx.x & 31) == 0) { sm[threadIdx.x >> 5] = m; ss[threadIdx.x >> 5] = s; st[threadIdx.x >> 5] = tsum; }
  __syncthreads();
  if (threadIdx.x < 32) {
    int nw = blockDim.x >> 5;
    m = threadIdx.x < nw ? sm[threadIdx.x] : -INFINITY;
    s = threadIdx.x < nw ? ss[threadIdx.x] : 0.f;
    tsum = threadIdx.x < nw ? st[threadIdx.x] : 0.f;
    for (int o = 16; o > 0; o >>= 1) {
      float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, s, o);
      online_combine(m, s, m2, s2);
      tsum += __shfl_xor_sync(0xffffffffu, tsum, o);
    }
    if (threadIdx.x == 0) { sm[0] = m; ss[0] = s; st[0] = tsum; }
  }
  __syncthreads();
  m = sm[0]; s = ss[0]; tsum = st[0];
  const float inv_s = 1.f / s;
  float l = 0.f;
  for (int c = threadIdx.x; c < V; c += blockDim.x) {
    float pr = __expf(lf(xr + c) - m) * inv_s;
    float t = lf(tr + c);
    if (t != 0.f) l -= t * logf(fmaxf(pr, 1e-12f));
    if (dlogits) sf(dlogits + row * (long long)V + c, (pr * tsum - t) * grad_scale);
  }
  for (int o = 16; o > 0; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
  if ((threadIdx.x & 31) == 0 && loss_sum) atomicAdd(loss_sum, l * loss_scale);
}

// kind: 0 MSE, 1 L1, 2 Huber(delta), 3 BCE (probabilities), 4 BCE-with-logits.
// loss_sum += sum_i l_i * loss_scale ;  grad_i = dl_i/dpred_i * grad_scale
template <typename T>
__global__ void pointwise_loss_kernel(const T* __restrict__ pred, const T* __restrict__ target, T* __restrict__ grad,
                                      float* __restrict__ loss_sum, long long n, int kind, float delta,
                                      float grad_scale, float loss_scale) {
  float acc = 0.f;
  long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  long long stride = (long long)gridDim.x * blockDim.x;
  for (; i < n; i += stride) {
    float p = lf(pred + i), t = lf(target + i), l, g;
    float d = p - t;
    switch (kind) {
      case 0: l = d * d; g = 2.f * d; break;
      case 1: l = fabsf(d); g = d > 0.f ? 1.f : (d < 0.f ? -1.f : 0.f); break;
      case 2: if (fabsf(d) <= delta) { l = 0.5f * d * d; g = d; } else { l = delta * (fabsf(d) - 0.5f * delta); g = d > 0.f ? delta : -delta; } break;
      case 3: { float pc = fminf(fmaxf(p, 1e-12f), 1.f - 1e-12f); l = -(t * logf(pc) + (1.f - t) * logf(1.f - pc)); g = (pc - t) / (pc * (1.f - pc)); break; }
      default: { float mx = fmaxf(p, 0.f); l = mx - p * t + log1pf(__expf(-fabsf(p))); g = 1.f / (1.f + __expf(-p)) - t; break; }
    }
    acc += l;
    if (grad) sf(grad + i, g * grad_scale);
  }
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  __shared__ float sh[32];
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    acc = threadIdx.x < (blockDim.x >> 5) ? sh[threadIdx.x] : 0.f;
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (threadIdx.x == 0 && loss_sum) atomicAdd(loss_sum, acc * loss_scale);
  }
}

}  // namespace b200

using namespace b200;

extern "C" {

int b200_ce_label(const void* logits, const long long* labels, void* dlogits, float* loss_rows, float* loss_sum,
                  long long rows, int V, long long ld, float grad_scale, float loss_scale, int is_bf16,
                  cudaStream_t st) {
  if (rows <= 0) return 0;
  int block = V >= 8192 ? 512 : 256;
  if (is_bf16) ce_label_kernel<__nv_bfloat16><<<(unsigned)rows, block, 0, st>>>((const __nv_bfloat16*)logits, labels, (__nv_bfloat16*)dlogits, loss_rows, loss_sum, V, ld, grad_scale, loss_scale);
  else ce_label_kernel<float><<<(unsigned)rows, block, 0, st>>>((const float*)logits, labels, (float*)dlogits, loss_rows, loss_sum, V, ld, grad_scale, loss_scale);
  return (int)cudaGetLastError();
}

int b200_ce_dense(const void* logits, const void* target, void* dlogits, float* loss_sum, long long rows, int V,
                  float grad_scale, float loss_scale, int is_bf16, cudaStream_t st) {
  if (rows <= 0) return 0;
  int block = V >= 4096 ? 512 : (V >= 256 ? 256 : 64);
  if (is_bf16) ce_dense_kernel<__nv_bfloat16><<<(unsigned)rows, block, 0, st>>>((const __nv_bfloat16*)logits, (const __nv_bfloat16*)target, (__nv_bfloat16*)dlogits, loss_sum, V, grad_scale, loss_scale);
  else ce_dense_kernel<float><<<(unsigned)rows, block, 0, st>>>((const float*)logits, (const float*)target, (float*)dlogits, loss_sum, V, grad_scale, loss_scale);
  return (int)cudaGetLastError();
}

int b200_pointwise_loss(const void* pred, const void* target, void* grad, float* loss_sum, long long n, int kind,
                        float delta, float grad_scale, float loss_scale, int is_bf16, cudaStream_t st) {
  if (n <= 0) return 0;
  long long g = (n + 255) / 256; if (g > 148 * 8) g = 148 * 8;
  if (is_bf16) pointwise_loss_kernel<__nv_bfloat16><<<(int)g, 256, 0, st>>>((const __nv_bfloat16*)pred, (const __nv_bfloat16*)target, (__nv_bfloat16*)grad, loss_sum, n, kind, delta, grad_scale, loss_scale);
  else pointwise_loss_kernel<float><<<(int)g, 256, 0, st>>>((const float*)pred, (const float*)target, (float*)grad, loss_sum, n, kind, delta, grad_scale, loss_scale);
  return (int)cudaGetLastError();
}

}  // extern "C"
