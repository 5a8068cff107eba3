// Quantisation kernels: the producers and consumers around the 8-bit tensor-core GEMM kinds.
//
//   rows      : per-row symmetric int8 (absmax/127) and fp8-e4m3 (absmax/448) quantisation of
//               weights and of activations on the fly (rust-nn src/int8.rs:24-52 for the weight side)
//   group     : group-wise INT8 / INT4 / NF4 / NVFP4(E2M1) / Q4_0 / Q8_0 quantise + dequantise with the
//               reference's tables, scales and nibble order (src/quantize.rs:97-215, 289-612)
//   ternary   : {-1,0,+1} with threshold 0.7*mean|w| and scale mean|w| per row, 16 codes per u32
//               (src/ternary.rs:46-137), and the unpack that feeds the GEMM
//   rotor     : RotorQuant fake-quantisation: rotate 3-groups, quantise, rotate back (src/quant.rs:150-196)
//   csr spmm  : C = S * B for a CSR matrix (src/compression.rs:134-152)
//
// Rounding is round-half-away-from-zero (roundf), as Rust's f32::round.
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <cstdint>

namespace {

template <typename T> __device__ __forceinline__ float ldf(const T* p, long long i);
template <> __device__ __forceinline__ float ldf<float>(const float* p, long long i) { return p[i]; }
template <> __device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16* p, long long i) { return __bfloat162float(p[i]); }
template <typename T> __device__ __forceinline__ void stf(T* p, long long i, float v);
template <> __device__ __forceinline__ void stf<float>(float* p, long long i, float v) { p[i] = v; }
template <> __device__ __forceinline__ void stf<__nv_bfloat16>(__nv_bfloat16* p, long long i, float v) { p[i] = __float2bfloat16(v); }

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_add(float v) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
// block-wide reduction through shared memory; every thread gets the result
template <bool MAX>
__device__ __forceinline__ float block_reduce(float v, float* sh) {
  v = MAX ? warp_max(v) : warp_add(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (l == 0) sh[w] = v;
  __syncthreads();
  float r = (l < nw) ? sh[l] : (MAX ? 0.f : 0.f);
  r = MAX ? warp_max(r) : warp_add(r);
  return __shfl_sync(0xffffffffu, r, 0);
}

// ------------------------------------------------------------------ per-row int8 / e4m3
// mode 0: int8, scale = absmax/127 (1 when the row is zero); mode 1: e4m3, scale = absmax/448.
template <typename T>
__global__ void quant_rows_kernel(const T* __restrict__ x, long long ldx, int cols, uint8_t* __restrict__ q, long long ldq,
                                  float* __restrict__ scales, int mode) {
  __shared__ float sh[32];
  const long long r = blockIdx.x;
  const T* xr = x + r * ldx;
  float m = 0.f;
  for (int j = threadIdx.x; j < cols; j += blockDim.x) m = fmaxf(m, fabsf(ldf(xr, j)));
  m = block_reduce<true>(m, sh);
  const float qmax = mode == 0 ? 127.f : 448.f;
  const float scale = m > 0.f ? m / qmax : 1.f;
  if (threadIdx.x == 0) scales[r] = scale;
  uint8_t* qr = q + r * ldq;
  for (int j = threadIdx.x; j < cols; j += blockDim.x) {
    const float v = ldf(xr, j) / scale;
    if (mode == 0) {
      qr[j] = (uint8_t)(int8_t)fminf(fmaxf(roundf(v), -128.f), 127.f);
    } else {
      qr[j] = (uint8_t)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
    }
  }
}

// ------------------------------------------------------------------ group-wise formats
enum { Q_INT8 = 0, Q_INT4 = 1, Q_NF4 = 2, Q_NVFP4 = 3, Q_Q4_0 = 4, Q_Q8_0 = 5 };

__constant__ float c_nf4[16] = {-1.0f, -0.6961928f, -0.52507305f, -0.3949175f, -0.28444138f, -0.18477343f, -0.091050036f, 0.0f,
                                0.0795803f, 0.1609302f, 0.2461123f, 0.33791524f, 0.44070983f, 0.562617f, 0.72295684f, 1.0f};
__constant__ float c_fp4_mag[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};

// non-negative floats order like their bit patterns: absmax via atomicMax on uint32
template <typename T>
__global__ void group_absmax_kernel(const T* __restrict__ x, long long n, long long gs, uint32_t* __restrict__ absmax) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const bool in = i < n;
  const float a = in ? fabsf(ldf(x, i)) : 0.f;
  const long long g = in ? i / gs : -1;
  // whole warp inside one group: one atomic for the warp
  const long long g0 = __shfl_sync(0xffffffffu, g, 0), g31 = __shfl_sync(0xffffffffu, g, 31);
  if (g0 == g31 && g0 >= 0) {
    const float m = warp_max(a);
    if ((threadIdx.x & 31) == 0) atomicMax(absmax + g0, __float_as_uint(m));
  } else if (in) {
    atomicMax(absmax + g, __float_as_uint(a));
  }
}

__device__ __forceinline__ float group_scale(float m, int fmt) {
  switch (fmt) {
    case Q_INT8: case Q_Q8_0: return m > 0.f ? m / 127.f : 1.f;
    case Q_INT4: return m > 0.f ? m / 7.f : 1.f;
    case Q_NF4: return m > 0.f ? m : 1.f;
    case Q_NVFP4: return m > 0.f ? m / 6.f : 1.f;
    default: { const float s = m / -8.f; return s == 0.f ? 1.f : s; }   // Q4_0: the scale is negative
  }
}
__device__ __forceinline__ uint32_t quant_code(float v, float scale, int fmt) {
  const float t = v / scale;
  switch (fmt) {
    case Q_INT8: case Q_Q8_0: return (uint32_t)(uint8_t)(int8_t)fminf(fmaxf(roundf(t), -128.f), 127.f);
    case Q_INT4: case Q_Q4_0: return (uint32_t)((int)fminf(fmaxf(roundf(t), -8.f), 7.f)) & 0xFu;
    case Q_NF4: {
      uint32_t best = 0; float bd = INFINITY;
#pragma unroll
      for (int i = 0; i < 16; ++i) { const float d = fabsf(c_nf4[i] - t); if (d < bd) { bd = d; best = i; } }
      return best;
    }
    default: {   // NVFP4 (E2M1): sign bit 8, nearest magnitude, first minimum wins
      const float a = fabsf(t);
      uint32_t best = 0; float bd = INFINITY;
#pragma unroll
      for (int i = 0; i < 8; ++i) { const float d = fabsf(c_fp4_mag[i] - a); if (d < bd) { bd = d; best = i; } }
      return (t < 0.f ? 8u : 0u) | best;
    }
  }
}
__device__ __forceinline__ float dequant_code(uint32_t c, float scale, int fmt) {
  switch (fmt) {
    case Q_INT8: case Q_Q8_0: return (float)(int8_t)(uint8_t)c * scale;
    case Q_INT4: case Q_Q4_0: return (float)((c & 8u) ? (int)c - 16 : (int)c) * scale;
    case Q_NF4: return c_nf4[c & 15u] * scale;
    default: { const float m = c_fp4_mag[c & 7u]; return ((c & 8u) ? -m : m) * scale; }
  }
}

// One thread per PAIR of in-group elements (one output byte for the 4-bit formats, two for 8-bit).
// Group g's bytes start at g * ceil(gs/2) for 4-bit formats, g * gs for 8-bit ones.
template <typename T>
__global__ void group_quant_kernel(const T* __restrict__ x, long long n, long long gs, int fmt, const uint32_t* __restrict__ absmax,
                                   float* __restrict__ scales, uint8_t* __restrict__ data) {
  const long long pairs_per_group = (gs + 1) / 2;
  const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long g = t / pairs_per_group, jp = t % pairs_per_group;
  const long long i0 = g * gs + 2 * jp;
  if (i0 >= n) return;
  const float scale = group_scale(__uint_as_float(absmax[g]), fmt);
  if (jp == 0) scales[g] = scale;
  const bool has1 = (2 * jp + 1 < gs) && (i0 + 1 < n);
  const uint32_t c0 = quant_code(ldf(x, i0), scale, fmt);
  const uint32_t c1 = has1 ? quant_code(ldf(x, i0 + 1), scale, fmt) : 0u;
  if (fmt == Q_INT8 || fmt == Q_Q8_0) {
    data[i0] = (uint8_t)c0;
    if (has1) data[i0 + 1] = (uint8_t)c1;
  } else {
    data[g * pairs_per_group + jp] = (uint8_t)(c0 | (c1 << 4));
  }
}

template <typename T>
__global__ void group_dequant_kernel(const uint8_t* __restrict__ data, const float* __restrict__ scales, long long n, long long gs,
                                     int fmt, T* __restrict__ out) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const long long g = i / gs, j = i % gs;
  const float scale = scales[g];
  uint32_t c;
  if (fmt == Q_INT8 || fmt == Q_Q8_0) c = data[i];
  else {
    const uint8_t b = data[g * ((gs + 1) / 2) + j / 2];
    c = (j & 1) ? (b >> 4) & 0xFu : b & 0xFu;
  }
  stf(out, i, dequant_code(c, scale, fmt));
}

// ------------------------------------------------------------------ ternary
template <typename T>
__global__ void ternary_row_stats_kernel(const T* __restrict__ w, int cols, float* __restrict__ mean_abs, float* __restrict__ scales) {
  __shared__ float sh[32];
  const long long r = blockIdx.x;
  float s = 0.f;
  for (int j = threadIdx.x; j < cols; j += blockDim.x) s += fabsf(ldf(w, r * cols + j));
  s = block_reduce<false>(s, sh);
  if (threadIdx.x == 0) {
    const float m = s / (float)(cols > 0 ? cols : 1);
    mean_abs[r] = m;
    scales[r] = fmaxf(m, 1e-8f);
  }
}
// one thread per packed word (16 codes): 0 -> 0, +1 -> 1, -1 -> 2
template <typename T>
__global__ void ternary_pack_kernel(const T* __restrict__ w, long long numel, int cols, const float* __restrict__ mean_abs,
                                    uint32_t* __restrict__ packed) {
  const long long word = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long i0 = word * 16;
  if (i0 >= numel) return;
  uint32_t out = 0;
#pragma unroll
  for (int k = 0; k < 16; ++k) {
    const long long i = i0 + k;
    if (i < numel) {
      const float v = ldf(w, i);
      const float thr = 0.7f * mean_abs[i / cols];
      const uint32_t code = fabsf(v) < thr ? 0u : (v > 0.f ? 1u : 2u);
      out |= code << (2 * k);
    }
  }
  packed[word] = out;
}
// unpack to {-1,0,1} (scaled by the row's scale when `scales` is given)
template <typename T>
__global__ void ternary_unpack_kernel(const uint32_t* __restrict__ packed, long long numel, int cols, const float* __restrict__ scales,
                                      T* __restrict__ out) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= numel) return;
  const uint32_t code = (packed[i >> 4] >> ((i & 15) * 2)) & 3u;
  float v = code == 1u ? 1.f : (code == 2u ? -1.f : 0.f);
  if (scales) v *= scales[i / cols];
  stf(out, i, v);
}
// counts[0..2] = (+1, -1, 0)
__global__ void ternary_count_kernel(const uint32_t* __restrict__ packed, long long numel, unsigned long long* __restrict__ counts) {
  const long long word = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long i0 = word * 16;
  unsigned pos = 0, neg = 0, zero = 0;
  if (i0 < numel) {
    const uint32_t wv = packed[word];
    const int valid = (int)((numel - i0) < 16 ? (numel - i0) : 16);
    for (int k = 0; k < valid; ++k) {
      const uint32_t c = (wv >> (2 * k)) & 3u;
      pos += c == 1u; neg += c == 2u; zero += (c == 0u || c == 3u);
    }
  }
  pos = __reduce_add_sync(0xffffffffu, pos); neg = __reduce_add_sync(0xffffffffu, neg); zero = __reduce_add_sync(0xffffffffu, zero);
  if ((threadIdx.x & 31) == 0) {
    if (pos) atomicAdd(counts, (unsigned long long)pos);
    if (neg) atomicAdd(counts + 1, (unsigned long long)neg);
    if (zero) atomicAdd(counts + 2, (unsigned long long)zero);
  }
}

// ------------------------------------------------------------------ RotorQuant
// one thread per (row, 3-group): v' = R^T quant(R v); rot holds row-major 3x3 matrices
template <typename T>
__global__ void rotor_quant_kernel(const T* __restrict__ x, const float* __restrict__ rot, long long rows, int dim, int groups,
                                   float qmax, T* __restrict__ out) {
  const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= rows * groups) return;
  const long long r = t / groups; const int g = (int)(t % groups);
  const float* R = rot + 9 * g;
  float v[3];
#pragma unroll
  for (int k = 0; k < 3; ++k) v[k] = (3 * g + k < dim) ? ldf(x, r * dim + 3 * g + k) : 0.f;
  float rv[3];
#pragma unroll
  for (int a = 0; a < 3; ++a) rv[a] = R[3 * a] * v[0] + R[3 * a + 1] * v[1] + R[3 * a + 2] * v[2];
  const float m = fmaxf(fabsf(rv[0]), fmaxf(fabsf(rv[1]), fabsf(rv[2])));
  float o[3] = {v[0], v[1], v[2]};
  if (m >= 1e-12f) {
    const float scale = m / qmax;
#pragma unroll
    for (int a = 0; a < 3; ++a) rv[a] = fminf(fmaxf(roundf(rv[a] / scale), -qmax), qmax) * scale;
#pragma unroll
    for (int k = 0; k < 3; ++k) o[k] = R[k] * rv[0] + R[3 + k] * rv[1] + R[6 + k] * rv[2];
  }
#pragma unroll
  for (int k = 0; k < 3; ++k) if (3 * g + k < dim) stf(out, r * dim + 3 * g + k, o[k]);
}

// ------------------------------------------------------------------ CSR SpMM: C[m,n] = S[m,k] * B[k,n]
// one warp per (row, 32-column strip of C)
__global__ void csr_spmm_kernel(const float* __restrict__ vals, const int* __restrict__ col_idx, const int* __restrict__ row_ptr,
                                const float* __restrict__ B, float* __restrict__ C, int m, int n) {
  const int strips = (n + 31) / 32;
  const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (warp >= (long long)m * strips) return;
  const int r = (int)(warp / strips), j = (int)(warp % strips) * 32 + (threadIdx.x & 31);
  float acc = 0.f;
  const int e0 = row_ptr[r], e1 = row_ptr[r + 1];
  for (int e = e0; e < e1; ++e) {
    const float v = __ldg(vals + e);
    const int c = __ldg(col_idx + e);
    if (j < n) acc += v * __ldg(B + (long long)c * n + j);
  }
  if (j < n) C[(long long)r * n + j] = acc;
}

inline int blocks_for(long long n, int t) { return (int)((n + t - 1) / t); }

}  // namespace

extern "C" {

int b200_quant_rows(const void* x, int is_bf16, long long rows, int cols, long long ldx, void* q, long long ldq, float* scales,
                    int mode, cudaStream_t st) {
  if (rows <= 0 || cols <= 0) return 0;
  const int threads = cols >= 1024 ? 256 : 128;
  if (is_bf16) quant_rows_kernel<__nv_bfloat16><<<(unsigned)rows, threads, 0, st>>>((const __nv_bfloat16*)x, ldx, cols, (uint8_t*)q, ldq, scales, mode);
  else quant_rows_kernel<float><<<(unsigned)rows, threads, 0, st>>>((const float*)x, ldx, cols, (uint8_t*)q, ldq, scales, mode);
  return (int)cudaGetLastError();
}

// absmax: [groups] uint32 scratch, zeroed by this call
int b200_quant_group(const void* x, int is_bf16, long long n, long long gs, int fmt, uint32_t* absmax, float* scales, uint8_t* data,
                     cudaStream_t st) {
  if (n <= 0 || gs <= 0) return 0;
  const long long groups = (n + gs - 1) / gs;
  cudaError_t e = cudaMemsetAsync(absmax, 0, groups * sizeof(uint32_t), st);
  if (e != cudaSuccess) return (int)e;
  const long long pairs = groups * ((gs + 1) / 2);
  if (is_bf16) {
    group_absmax_kernel<__nv_bfloat16><<<blocks_for(n, 256), 256, 0, st>>>((const __nv_bfloat16*)x, n, gs, absmax);
    group_quant_kernel<__nv_bfloat16><<<blocks_for(pairs, 256), 256, 0, st>>>((const __nv_bfloat16*)x, n, gs, fmt, absmax, scales, data);
  } else {
    group_absmax_kernel<float><<<blocks_for(n, 256), 256, 0, st>>>((const float*)x, n, gs, absmax);
    group_quant_kernel<float><<<blocks_for(pairs, 256), 256, 0, st>>>((const float*)x, n, gs, fmt, absmax, scales, data);
  }
  return (int)cudaGetLastError();
}

int b200_dequant_group(const uint8_t* data, const float* scales, long long n, long long gs, int fmt, void* out, int out_bf16,
                       cudaStream_t st) {
  if (n <= 0 || gs <= 0) return 0;
  if (out_bf16) group_dequant_kernel<__nv_bfloat16><<<blocks_for(n, 256), 256, 0, st>>>(data, scales, n, gs, fmt, (__nv_bfloat16*)out);
  else group_dequant_kernel<float><<<blocks_for(n, 256), 256, 0, st>>>(data, scales, n, gs, fmt, (float*)out);
  return (int)cudaGetLastError();
}

int b200_ternary_quant(const void* w, int is_bf16, long long rows, int cols, float* mean_abs, float* scales, uint32_t* packed,
                       cudaStream_t st) {
  const long long numel = rows * cols;
  if (numel <= 0) return 0;
  const long long words = (numel + 15) / 16;
  if (is_bf16) {
    ternary_row_stats_kernel<__nv_bfloat16><<<(unsigned)rows, 256, 0, st>>>((const __nv_bfloat16*)w, cols, mean_abs, scales);
    ternary_pack_kernel<__nv_bfloat16><<<blocks_for(words, 256), 256, 0, st>>>((const __nv_bfloat16*)w, numel, cols, mean_abs, packed);
  } else {
    ternary_row_stats_kernel<float><<<(unsigned)rows, 256, 0, st>>>((const float*)w, cols, mean_abs, scales);
    ternary_pack_kernel<float><<<blocks_for(words, 256), 256, 0, st>>>((const float*)w, numel, cols, mean_abs, packed);
  }
  return (int)cudaGetLastError();
}

int b200_ternary_unpack(const uint32_t* packed, long long numel, int cols, const float* scales, void* out, int out_bf16, cudaStream_t st) {
  if (numel <= 0) return 0;
  if (out_bf16) ternary_unpack_kernel<__nv_bfloat16><<<blocks_for(numel, 256), 256, 0, st>>>(packed, numel, cols, scales, (__nv_bfloat16*)out);
  else ternary_unpack_kernel<float><<<blocks_for(numel, 256), 256, 0, st>>>(packed, numel, cols, scales, (float*)out);
  return (int)cudaGetLastError();
}

// counts: 3 x uint64, zeroed by this call
int b200_ternary_count(const uint32_t* packed, long long numel, unsigned long long* counts, cudaStream_t st) {
  cudaError_t e = cudaMemsetAsync(counts, 0, 3 * sizeof(unsigned long long), st);
  if (e != cudaSuccess) return (int)e;
  if (numel <= 0) return 0;
  ternary_count_kernel<<<blocks_for((numel + 15) / 16, 256), 256, 0, st>>>(packed, numel, counts);
  return (int)cudaGetLastError();
}

int b200_rotor_quant(const void* x, int is_bf16, const float* rot, long long rows, int dim, int groups, float qmax, void* out,
                     cudaStream_t st) {
  const long long n = rows * groups;
  if (n <= 0) return 0;
  if (is_bf16) rotor_quant_kernel<__nv_bfloat16><<<blocks_for(n, 256), 256, 0, st>>>((const __nv_bfloat16*)x, rot, rows, dim, groups, qmax, (__nv_bfloat16*)out);
  else rotor_quant_kernel<float><<<blocks_for(n, 256), 256, 0, st>>>((const float*)x, rot, rows, dim, groups, qmax, (float*)out);
  return (int)cudaGetLastError();
}

int b200_csr_spmm(const float* vals, const int* col_idx, const int* row_ptr, const float* B, float* C, int m, int n, cudaStream_t st) {
  if (m <= 0 || n <= 0) return 0;
  const long long warps = (long long)m * ((n + 31) / 32);
  csr_spmm_kernel<<<blocks_for(warps * 32, 256), 256, 0, st>>>(vals, col_idx, row_ptr, B, C, m, n);
  return (int)cudaGetLastError();
}

}  // extern "C"
