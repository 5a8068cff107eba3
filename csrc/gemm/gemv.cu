// G2: GEMV and the level-1 BLAS routines (rust-nn src/blas.rs:597-710).
//
//   y = alpha * op(A) x + beta * y        A: [m, n] row-major, fp32 or bf16; x, y fp32
//
// A matrix-vector product moves m*n elements for 2*m*n flops, so it is bound by HBM bandwidth and
// the tensor cores have nothing to add: the kernels below only try to keep every load a full
// 16-byte vector and every warp's accesses contiguous.
//   NoTrans : one warp per row; lanes stride over the row with 16-byte loads, shuffle reduction.
//   Trans   : y[j] = sum_i A[i][j] x[i]; a block owns a strip of 128 columns (one column per
//             thread, coalesced across the warp) and a slab of rows; slabs combine with atomics.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cstdint>

namespace {

__device__ __forceinline__ float warp_add(float v) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

template <typename T> struct Vec;
template <> struct Vec<float> {
  static constexpr int N = 4;
  __device__ static __forceinline__ void load(const float* p, float (&o)[4]) {
    const float4 v = __ldg(reinterpret_cast<const float4*>(p));
    o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
  }
  __device__ static __forceinline__ float one(const float* p) { return __ldg(p); }
};
template <> struct Vec<__nv_bfloat16> {
  static constexpr int N = 8;
  __device__ static __forceinline__ void load(const __nv_bfloat16* p, float (&o)[8]) {
    const uint4 v = __ldg(reinterpret_cast<const uint4*>(p));
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) { o[2 * i] = __uint_as_float(w[i] << 16); o[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u); }
  }
  __device__ static __forceinline__ float one(const __nv_bfloat16* p) { return __bfloat162float(*p); }
};

template <typename T>
__global__ void gemv_n_kernel(const T* __restrict__ A, long long lda, const float* __restrict__ x, float* __restrict__ y, int m, int n,
                              float alpha, float beta, int vec_ok) {
  constexpr int V = Vec<T>::N;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= m) return;
  const T* a = A + (long long)row * lda;
  float acc = 0.f;
  int j0 = 0;
  if (vec_ok) {
    const int nv = n / V;
    for (int c = lane; c < nv; c += 32) {
      float av[V];
      Vec<T>::load(a + c * V, av);
#pragma unroll
      for (int k = 0; k < V; k += 4) {
        const float4 xv = __ldg(reinterpret_cast<const float4*>(x + c * V + k));
        acc += av[k] * xv.x + av[k + 1] * xv.y + av[k + 2] * xv.z + av[k + 3] * xv.w;
      }
    }
    j0 = nv * V;
  }
  for (int j = j0 + lane; j < n; j += 32) acc += Vec<T>::one(a + j) * __ldg(x + j);
  acc = warp_add(acc);
  if (lane == 0) y[row] = alpha * acc + (beta == 0.f ? 0.f : beta * y[row]);
}

// y must already hold beta*y (scaled by the launcher); partial sums are added atomically
template <typename T>
__global__ void gemv_t_kernel(const T* __restrict__ A, long long lda, const float* __restrict__ x, float* __restrict__ y, int m, int n,
                              float alpha, int rows_per_block) {
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  const int r0 = blockIdx.y * rows_per_block;
  const int r1 = min(r0 + rows_per_block, m);
  if (j >= n) return;
  float acc = 0.f;
#pragma unroll 4
  for (int i = r0; i < r1; ++i) acc += Vec<T>::one(A + (long long)i * lda + j) * __ldg(x + i);
  atomicAdd(y + j, alpha * acc);
}

__global__ void scale_kernel(float* y, long long n, float s) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) y[i] = (s == 0.f) ? 0.f : y[i] * s;
}

// out[0] += sum x[i*incx] * y[i*incy]   (out zeroed by the launcher)
__global__ void dot_kernel(const float* __restrict__ x, long long incx, const float* __restrict__ y, long long incy, long long n, float* out) {
  float acc = 0.f;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    acc += x[i * incx] * y[i * incy];
  acc = warp_add(acc);
  __shared__ float sh[32];
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < (blockDim.x >> 5) ? sh[threadIdx.x] : 0.f;
    v = warp_add(v);
    if (threadIdx.x == 0) atomicAdd(out, v);
  }
}
__global__ void axpy_kernel(float alpha, const float* __restrict__ x, float* __restrict__ y, long long n) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) y[i] += alpha * x[i];
}
__global__ void sqrt_inplace_kernel(float* v) { v[0] = sqrtf(v[0]); }

inline int blocks_for(long long n, int t) { return (int)((n + t - 1) / t); }

}  // namespace

extern "C" {

int b200_gemv(const void* A, int a_bf16, long long lda, int trans, const float* x, float* y, int m, int n, float alpha, float beta,
              cudaStream_t st) {
  if (m <= 0 || n <= 0) return 0;
  if (!trans) {
    const int es = a_bf16 ? 2 : 4;
    const int vec_ok = ((uintptr_t)A % 16 == 0) && ((lda * es) % 16 == 0) && ((uintptr_t)x % 16 == 0);
    const int warps = 8;
    if (a_bf16) gemv_n_kernel<__nv_bfloat16><<<blocks_for(m, warps), warps * 32, 0, st>>>((const __nv_bfloat16*)A, lda, x, y, m, n, alpha, beta, vec_ok);
    else gemv_n_kernel<float><<<blocks_for(m, warps), warps * 32, 0, st>>>((const float*)A, lda, x, y, m, n, alpha, beta, vec_ok);
  } else {
    // op(A) = A^T: output has n entries, reduction over the m rows
    scale_kernel<<<blocks_for(n, 256), 256, 0, st>>>(y, n, beta);
    int slabs = (int)((148LL * 8 * 128 + n - 1) / n);          // enough blocks to fill the machine
    if (slabs < 1) slabs = 1;
    if (slabs > (m + 63) / 64) slabs = (m + 63) / 64;
    if (slabs < 1) slabs = 1;
    const int rows_per_block = (m + slabs - 1) / slabs;
    dim3 grid(blocks_for(n, 128), (m + rows_per_block - 1) / rows_per_block);
    if (a_bf16) gemv_t_kernel<__nv_bfloat16><<<grid, 128, 0, st>>>((const __nv_bfloat16*)A, lda, x, y, m, n, alpha, rows_per_block);
    else gemv_t_kernel<float><<<grid, 128, 0, st>>>((const float*)A, lda, x, y, m, n, alpha, rows_per_block);
  }
  return (int)cudaGetLastError();
}

// out: one device float. sqrt_result != 0 gives the 2-norm when x == y.
int b200_dot(const float* x, long long incx, const float* y, long long incy, long long n, float* out, int sqrt_result, cudaStream_t st) {
  cudaError_t e = cudaMemsetAsync(out, 0, sizeof(float), st);
  if (e != cudaSuccess) return (int)e;
  if (n > 0) {
    int grid = blocks_for(n, 256);
    if (grid > 148 * 8) grid = 148 * 8;
    dot_kernel<<<grid, 256, 0, st>>>(x, incx, y, incy, n, out);
  }
  if (sqrt_result) sqrt_inplace_kernel<<<1, 1, 0, st>>>(out);
  return (int)cudaGetLastError();
}

int b200_axpy(float alpha, const float* x, float* y, long long n, cudaStream_t st) {
  if (n <= 0) return 0;
  axpy_kernel<<<blocks_for(n, 256), 256, 0, st>>>(alpha, x, y, n);
  return (int)cudaGetLastError();
}

int b200_scal(float alpha, float* x, long long n, cudaStream_t st) {
  if (n <= 0) return 0;
  scale_kernel<<<blocks_for(n, 256), 256, 0, st>>>(x, n, alpha);
  return (int)cudaGetLastError();
}

}  // extern "C"
