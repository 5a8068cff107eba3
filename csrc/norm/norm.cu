// N1 LayerNorm forward/backward (last axis, eps inside the sqrt, biased variance) and
// N2 BatchNorm1D forward/backward with the full gradient and running statistics.
// Math restates rust-nn src/tensor.rs:1013-1062 (forward), 1904-2001 (backward) and
// src/nn.rs:342-388 (batch statistics, biased variance, eps 1e-5).
//
// LayerNorm: one warp per row, rows in a grid-stride loop; x is read once from HBM (the second
// pass hits L1), statistics are fp32, gamma/beta are fp32. dgamma/dbeta are reduced in shared
// memory per block and flushed with one fp32 atomic per column per block.
#include <cuda_runtime.h>
#include "../common/launch.cuh"
#include <cuda_bf16.h>
#include <cstdint>

namespace b200 {

template <typename T> __device__ __forceinline__ float ldf(const T* p);
template <> __device__ __forceinline__ float ldf<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void stf(T* p, float v);
template <> __device__ __forceinline__ void stf<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void stf<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16(v); }

__device__ __forceinline__ float wsum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// two elements per lane per step -> 128-byte (bf16) / 256-byte (f32) warp transactions
template <typename T> struct Pair;
template <> struct Pair<float> { using V = float2;
  static __device__ __forceinline__ float2 ld(const float* p) { return *reinterpret_cast<const float2*>(p); }
  static __device__ __forceinline__ void st(float* p, float a, float b) { *reinterpret_cast<float2*>(p) = make_float2(a, b); } };
template <> struct Pair<__nv_bfloat16> { using V = __nv_bfloat162;
  static __device__ __forceinline__ float2 ld(const __nv_bfloat16* p) { return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p)); }
  static __device__ __forceinline__ void st(__nv_bfloat16* p, float a, float b) { *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b); } };

template <typename T>
__global__ void layernorm_fwd_kernel(const T* __restrict__ x, const float* __restrict__ gamma,
                                     const float* __restrict__ beta, T* __restrict__ y, float* __restrict__ mean_out,
                                     float* __restrict__ rstd_out, long long rows, int d, float eps) {
  const int lane = threadIdx.x & 31;
  const int warps_per_block = blockDim.x >> 5;
  long long row = (long long)blockIdx.x * warps_per_block + (threadIdx.x >> 5);
  const long long row_stride = (long long)gridDim.x * warps_per_block;
  const bool even = (d % 2 == 0);
  for (; row < rows; row += row_stride) {
    const T* xr = x + row * d;
    float s = 0.f;
    if (even) { for (int c = 2 * lane; c < d; c += 64) { float2 v = Pair<T>::ld(xr + c); s += v.x + v.y; } }
    else { for (int c = lane; c < d; c += 32) s += ldf(xr + c); }
    const float mean = wsum(s) / d;
    float q = 0.f;
    if (even) { for (int c = 2 * lane; c < d; c += 64) { float2 v = Pair<T>::ld(xr + c); float a = v.x - mean, b = v.y - mean; q += a * a + b * b; } }
    else { for (int c = lane; c < d; c += 32) { float a = ldf(xr + c) - mean; q += a * a; } }
    const float rstd = rsqrtf(wsum(q) / d + eps);
    T* yr = y + row * d;
    if (even) {
      for (int c = 2 * lane; c < d; c += 64) {
        float2 v = Pair<T>::ld(xr + c);
        float2 g = *reinterpret_cast<const float2*>(gamma + c);
        float2 b = *reinterpret_cast<const float2*>(beta + c);
        Pair<T>::st(yr + c, (v.x - mean) * rstd * g.x + b.x, (v.y - mean) * rstd * g.y + b.y);
      }
    } else {
      for (int c = lane; c < d; c += 32) stf(yr + c, (ldf(xr + c) - mean) * rstd * gamma[c] + beta[c]);
    }
    if (lane == 0) { if (mean_out) mean_out[row] = mean; if (rstd_out) rstd_out[row] = rstd; }
  }
}

// bf16 rows whose length is a multiple of 256: the row lives in registers (8 contiguous columns per lane and
// 256-column chunk, one 16-byte load each), so x is read once and mean / variance / output need no second pass.
// J2 16-byte pieces per lane and W warps per row: d = 256 * J2 * W. With W > 1 the warps of a row meet twice per row
// in shared memory (mean, then variance); every warp of the block runs the same number of iterations so that the
// block-wide barriers line up.
template <int J2, int W>
__global__ void __launch_bounds__(256)
layernorm_fwd_vec_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ gamma, const float* __restrict__ beta,
                         __nv_bfloat16* __restrict__ y, float* __restrict__ mean_out, float* __restrict__ rstd_out,
                         long long rows, int d, float eps,
                         const __nv_bfloat16* __restrict__ res = nullptr, __nv_bfloat16* __restrict__ sum_out = nullptr) {
  // with `res`: the normalised row is x + res (rounded to bf16 first, so that it equals what `sum_out` stores and what
  // the backward pass will read); `sum_out` receives that sum. This is the residual add of the layer before, moved
  // out of its GEMM epilogue.
  __shared__ float red[2][2][8];              // [row parity][mean | variance][warp]
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int groups_per_block = (blockDim.x >> 5) / W, grp = warp / W, wi = warp % W;
  float gam[J2][8], bet[J2][8];
#pragma unroll
  for (int j = 0; j < J2; ++j) {
    const int c = 8 * lane + 256 * (j * W + wi);
    const float4 g0 = *reinterpret_cast<const float4*>(gamma + c), g1 = *reinterpret_cast<const float4*>(gamma + c + 4);
    const float4 b0 = *reinterpret_cast<const float4*>(beta + c), b1 = *reinterpret_cast<const float4*>(beta + c + 4);
    gam[j][0] = g0.x; gam[j][1] = g0.y; gam[j][2] = g0.z; gam[j][3] = g0.w; gam[j][4] = g1.x; gam[j][5] = g1.y; gam[j][6] = g1.z; gam[j][7] = g1.w;
    bet[j][0] = b0.x; bet[j][1] = b0.y; bet[j][2] = b0.z; bet[j][3] = b0.w; bet[j][4] = b1.x; bet[j][5] = b1.y; bet[j][6] = b1.z; bet[j][7] = b1.w;
  }
  const float inv_d = 1.f / d;
  const long long row_stride = (long long)gridDim.x * groups_per_block;
  const long long n_iter = (rows + row_stride - 1) / row_stride;
  for (long long it = 0; it < n_iter; ++it) {
    const long long row = it * row_stride + (long long)blockIdx.x * groups_per_block + grp;
    const bool valid = row < rows;
    if (W == 1 && !valid) break;
    const __nv_bfloat16* xr = x + row * d;
    uint4 xu[J2];
#pragma unroll
    for (int j = 0; j < J2; ++j) xu[j] = valid ? __ldg(reinterpret_cast<const uint4*>(xr + 8 * lane + 256 * (j * W + wi))) : make_uint4(0u, 0u, 0u, 0u);
    float v[J2][8];
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < J2; ++j) {
      const uint32_t w[4] = {xu[j].x, xu[j].y, xu[j].z, xu[j].w};
#pragma unroll
      for (int i = 0; i < 4; ++i) { v[j][2 * i] = __uint_as_float(w[i] << 16); v[j][2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u); }
      if (res != nullptr) {
        const int c = 8 * lane + 256 * (j * W + wi);
        const uint4 ru = valid ? __ldg(reinterpret_cast<const uint4*>(res + row * d + c)) : make_uint4(0u, 0u, 0u, 0u);
        const uint32_t rw[4] = {ru.x, ru.y, ru.z, ru.w};
        uint32_t ow[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const __nv_bfloat162 t = __floats2bfloat162_rn(v[j][2 * i] + __uint_as_float(rw[i] << 16), v[j][2 * i + 1] + __uint_as_float(rw[i] & 0xffff0000u));
          ow[i] = *reinterpret_cast<const uint32_t*>(&t);
          v[j][2 * i] = __low2float(t); v[j][2 * i + 1] = __high2float(t);
        }
        if (valid && sum_out != nullptr) *reinterpret_cast<uint4*>(sum_out + row * d + c) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) s += v[j][e];
    }
    s = wsum(s);
    if constexpr (W > 1) {
      if (lane == 0) red[it & 1][0][warp] = s;
      __syncthreads();
      s = 0.f;
#pragma unroll
      for (int k = 0; k < W; ++k) s += red[it & 1][0][grp * W + k];
    }
    const float mean = s * inv_d;
    float q = 0.f;
#pragma unroll
    for (int j = 0; j < J2; ++j)
#pragma unroll
      for (int e = 0; e < 8; ++e) { const float a = v[j][e] - mean; q += a * a; }
    q = wsum(q);
    if constexpr (W > 1) {
      if (lane == 0) red[it & 1][1][warp] = q;
      __syncthreads();
      q = 0.f;
#pragma unroll
      for (int k = 0; k < W; ++k) q += red[it & 1][1][grp * W + k];
      if (!valid) continue;
    }
    const float rstd = rsqrtf(q * inv_d + eps);
    __nv_bfloat16* yr = y + row * d;
#pragma unroll
    for (int j = 0; j < J2; ++j) {
      float o[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = (v[j][e] - mean) * rstd * gam[j][e] + bet[j][e];
      __nv_bfloat162 t0 = __floats2bfloat162_rn(o[0], o[1]), t1 = __floats2bfloat162_rn(o[2], o[3]);
      __nv_bfloat162 t2 = __floats2bfloat162_rn(o[4], o[5]), t3 = __floats2bfloat162_rn(o[6], o[7]);
      uint4 ou;
      ou.x = *reinterpret_cast<uint32_t*>(&t0); ou.y = *reinterpret_cast<uint32_t*>(&t1);
      ou.z = *reinterpret_cast<uint32_t*>(&t2); ou.w = *reinterpret_cast<uint32_t*>(&t3);
      *reinterpret_cast<uint4*>(yr + 8 * lane + 256 * (j * W + wi)) = ou;
    }
    if (lane == 0 && wi == 0) { if (mean_out) mean_out[row] = mean; if (rstd_out) rstd_out[row] = rstd; }
  }
}

template <typename T>
__global__ void layernorm_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x, const float* __restrict__ gamma,
                                     const float* __restrict__ mean_in, const float* __restrict__ rstd_in,
                                     T* __restrict__ dx, float* __restrict__ dgamma, float* __restrict__ dbeta,
                                     const T* __restrict__ dres, long long rows, int d) {
  extern __shared__ float sh[];   // [2*d]: dgamma partial, dbeta partial
  float* s_dg = sh; float* s_db = sh + d;
  for (int c = threadIdx.x; c < 2 * d; c += blockDim.x) sh[c] = 0.f;
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int warps_per_block = blockDim.x >> 5;
  long long row = (long long)blockIdx.x * warps_per_block + (threadIdx.x >> 5);
  const long long row_stride = (long long)gridDim.x * warps_per_block;
  for (; row < rows; row += row_stride) {
    const T* xr = x + row * d; const T* gr = dy + row * d;
    const float mean = mean_in[row], rstd = rstd_in[row];
    float s1 = 0.f, s2 = 0.f;
    for (int c = lane; c < d; c += 32) {
      float xh = (ldf(xr + c) - mean) * rstd;
      float g = ldf(gr + c);
      float gg = g * gamma[c];
      s1 += gg; s2 += gg * xh;
      atomicAdd(&s_dg[c], g * xh);
      atomicAdd(&s_db[c], g);
    }
    s1 = wsum(s1) / d; s2 = wsum(s2) / d;
    T* dxr = dx + row * d;
    for (int c = lane; c < d; c += 32) {
      float xh = (ldf(xr + c) - mean) * rstd;
      float gg = ldf(gr + c) * gamma[c];
      float out = rstd * (gg - s1 - xh * s2);
      if (dres) out += ldf(dres + row * d + c);   // gradient arriving through the residual branch
      stf(dxr + c, out);
    }
  }
  __syncthreads();
  for (int c = threadIdx.x; c < d; c += blockDim.x) {
    atomicAdd(dgamma + c, s_dg[c]);
    atomicAdd(dbeta + c, s_db[c]);
  }
}

// Register-accumulating variant for even d <= 64*J: lane l owns the column pairs {2l + 64j}, so the
// per-column dgamma/dbeta partial sums of every row a warp processes stay in that lane's registers;
// x and dy are read exactly once. Warps of a block are combined through shared memory, blocks with
// one fp32 atomic per column.
template <typename T, int J>
__global__ void __launch_bounds__(256)
layernorm_bwd_reg_kernel(const T* __restrict__ dy, const T* __restrict__ x, const float* __restrict__ gamma,
                         const float* __restrict__ mean_in, const float* __restrict__ rstd_in, T* __restrict__ dx,
                         float* __restrict__ dgamma, float* __restrict__ dbeta, const T* __restrict__ dres,
                         long long rows, int d) {
  extern __shared__ float sh[];   // [warps][2][d]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int warps_per_block = blockDim.x >> 5;
  float2 gam[J], adg[J], adb[J];
#pragma unroll
  for (int j = 0; j < J; ++j) {
    const int c = 2 * lane + 64 * j;
    gam[j] = c < d ? *reinterpret_cast<const float2*>(gamma + c) : make_float2(0.f, 0.f);
    adg[j] = make_float2(0.f, 0.f); adb[j] = make_float2(0.f, 0.f);
  }
  const float inv_d = 1.f / d;
  long long row = (long long)blockIdx.x * warps_per_block + warp;
  const long long row_stride = (long long)gridDim.x * warps_per_block;
  for (; row < rows; row += row_stride) {
    const T* xr = x + row * d; const T* gr = dy + row * d;
    const float mean = mean_in[row], rstd = rstd_in[row];
    float2 xh[J], g[J];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int j = 0; j < J; ++j) {
      const int c = 2 * lane + 64 * j;
      if (c < d) {
        const float2 xv = Pair<T>::ld(xr + c);
        g[j] = Pair<T>::ld(gr + c);
        xh[j] = make_float2((xv.x - mean) * rstd, (xv.y - mean) * rstd);
      } else { g[j] = make_float2(0.f, 0.f); xh[j] = make_float2(0.f, 0.f); }
      const float g0 = g[j].x * gam[j].x, g1 = g[j].y * gam[j].y;
      s1 += g0 + g1; s2 += g0 * xh[j].x + g1 * xh[j].y;
      adg[j].x += g[j].x * xh[j].x; adg[j].y += g[j].y * xh[j].y;
      adb[j].x += g[j].x; adb[j].y += g[j].y;
    }
    s1 = wsum(s1) * inv_d; s2 = wsum(s2) * inv_d;
    T* dxr = dx + row * d;
#pragma unroll
    for (int j = 0; j < J; ++j) {
      const int c = 2 * lane + 64 * j;
      if (c < d) {
        float o0 = rstd * (g[j].x * gam[j].x - s1 - xh[j].x * s2);
        float o1 = rstd * (g[j].y * gam[j].y - s1 - xh[j].y * s2);
        if (dres) { const float2 rr = Pair<T>::ld(dres + row * d + c); o0 += rr.x; o1 += rr.y; }
        Pair<T>::st(dxr + c, o0, o1);
      }
    }
  }
  float* my = sh + (size_t)warp * 2 * d;
#pragma unroll
  for (int j = 0; j < J; ++j) {
    const int c = 2 * lane + 64 * j;
    if (c < d) { my[c] = adg[j].x; my[c + 1] = adg[j].y; my[d + c] = adb[j].x; my[d + c + 1] = adb[j].y; }
  }
  __syncthreads();
  for (int c = threadIdx.x; c < 2 * d; c += blockDim.x) {
    float acc = 0.f;
    for (int w = 0; w < warps_per_block; ++w) acc += sh[(size_t)w * 2 * d + c];
    atomicAdd(c < d ? dgamma + c : dbeta + (c - d), acc);
  }
}

// bf16 rows whose length is a multiple of 256: every lane owns 8 contiguous columns per 256-column chunk and
// moves them with one 16-byte load / store (4x fewer memory instructions than the 2-column variant above).
// SUMS: the kernel also accumulates the column sums of `dres` and of its own output into `sum_dres` / `sum_dx` (fp32 [d],
// added to). In a pre-norm transformer block those are the bias gradients of the two projections whose outputs join
// the residual stream on either side of this LayerNorm, so two column-sum kernels (and two more passes over
// [rows, d] gradients) disappear.
template <int J2, int W, bool SUMS = false>
__global__ void __launch_bounds__(256)
layernorm_bwd_vec_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x, const float* __restrict__ gamma,
                         const float* __restrict__ mean_in, const float* __restrict__ rstd_in, __nv_bfloat16* __restrict__ dx,
                         float* __restrict__ dgamma, float* __restrict__ dbeta, const __nv_bfloat16* __restrict__ dres,
                         long long rows, int d, float* __restrict__ sum_dres = nullptr, float* __restrict__ sum_dx = nullptr) {
  constexpr int NS = SUMS ? 4 : 2;
  extern __shared__ float sh[];   // [row groups][NS][d]
  __shared__ float red[2][2][8];  // [row parity][s1 | s2][warp]
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int groups_per_block = (blockDim.x >> 5) / W, grp = warp / W, wi = warp % W;
  float gam[J2][8], adg[J2][8], adb[J2][8];
  float adr[SUMS ? J2 : 1][8], ado[SUMS ? J2 : 1][8];
#pragma unroll
  for (int j = 0; j < J2; ++j) {
    const int c = 8 * lane + 256 * (j * W + wi);
    const float4 g0 = *reinterpret_cast<const float4*>(gamma + c), g1 = *reinterpret_cast<const float4*>(gamma + c + 4);
    gam[j][0] = g0.x; gam[j][1] = g0.y; gam[j][2] = g0.z; gam[j][3] = g0.w; gam[j][4] = g1.x; gam[j][5] = g1.y; gam[j][6] = g1.z; gam[j][7] = g1.w;
#pragma unroll
    for (int e = 0; e < 8; ++e) { adg[j][e] = 0.f; adb[j][e] = 0.f; if (SUMS) { adr[j][e] = 0.f; ado[j][e] = 0.f; } }
  }
  const float inv_d = 1.f / d;
  auto unpack8 = [](const uint4& u, float (&o)[8]) {
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) { o[2 * i] = __uint_as_float(w[i] << 16); o[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u); }
  };
  const long long row_stride = (long long)gridDim.x * groups_per_block;
  const long long n_iter = (rows + row_stride - 1) / row_stride;
  for (long long it = 0; it < n_iter; ++it) {
    const long long row = it * row_stride + (long long)blockIdx.x * groups_per_block + grp;
    const bool valid = row < rows;
    if (W == 1 && !valid) break;
    const __nv_bfloat16* xr = x + row * d; const __nv_bfloat16* gr = dy + row * d;
    uint4 xu[J2], gu[J2], ru[J2];
#pragma unroll
    for (int j = 0; j < J2; ++j) {            // all loads of the row first: maximum memory-level parallelism
      const int c = 8 * lane + 256 * (j * W + wi);
      xu[j] = gu[j] = ru[j] = make_uint4(0u, 0u, 0u, 0u);
      if (valid) {
        xu[j] = __ldg(reinterpret_cast<const uint4*>(xr + c));
        gu[j] = __ldg(reinterpret_cast<const uint4*>(gr + c));
        if (dres) ru[j] = __ldg(reinterpret_cast<const uint4*>(dres + row * d + c));
      }
    }
    const float mean = valid ? mean_in[row] : 0.f, rstd = valid ? rstd_in[row] : 0.f;
    float xh[J2][8], g[J2][8];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int j = 0; j < J2; ++j) {
      float xv[8];
      unpack8(xu[j], xv); unpack8(gu[j], g[j]);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        xh[j][e] = (xv[e] - mean) * rstd;
        const float gg = g[j][e] * gam[j][e];
        s1 += gg; s2 += gg * xh[j][e];
        adg[j][e] += g[j][e] * xh[j][e];
        adb[j][e] += g[j][e];
      }
    }
    s1 = wsum(s1); s2 = wsum(s2);
    if constexpr (W > 1) {
      if (lane == 0) { red[it & 1][0][warp] = s1; red[it & 1][1][warp] = s2; }
      __syncthreads();
      s1 = s2 = 0.f;
#pragma unroll
      for (int k = 0; k < W; ++k) { s1 += red[it & 1][0][grp * W + k]; s2 += red[it & 1][1][grp * W + k]; }
      if (!valid) continue;
    }
    s1 *= inv_d; s2 *= inv_d;
    __nv_bfloat16* dxr = dx + row * d;
#pragma unroll
    for (int j = 0; j < J2; ++j) {
      const int c = 8 * lane + 256 * (j * W + wi);
      float o[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = rstd * (g[j][e] * gam[j][e] - s1 - xh[j][e] * s2);
      if (dres) {
        float rr[8];
        unpack8(ru[j], rr);
#pragma unroll
        for (int e = 0; e < 8; ++e) { o[e] += rr[e]; if (SUMS) adr[j][e] += rr[e]; }
      }
      if (SUMS) {
#pragma unroll
        for (int e = 0; e < 8; ++e) ado[j][e] += o[e];
      }
      uint4 ou;
      __nv_bfloat162 t0 = __floats2bfloat162_rn(o[0], o[1]), t1 = __floats2bfloat162_rn(o[2], o[3]);
      __nv_bfloat162 t2 = __floats2bfloat162_rn(o[4], o[5]), t3 = __floats2bfloat162_rn(o[6], o[7]);
      ou.x = *reinterpret_cast<uint32_t*>(&t0); ou.y = *reinterpret_cast<uint32_t*>(&t1);
      ou.z = *reinterpret_cast<uint32_t*>(&t2); ou.w = *reinterpret_cast<uint32_t*>(&t3);
      *reinterpret_cast<uint4*>(dxr + c) = ou;
    }
  }
  float* my = sh + (size_t)grp * NS * d;
#pragma unroll
  for (int j = 0; j < J2; ++j) {
    const int c = 8 * lane + 256 * (j * W + wi);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      my[c + e] = adg[j][e]; my[d + c + e] = adb[j][e];
      if (SUMS) { my[2 * d + c + e] = adr[j][e]; my[3 * d + c + e] = ado[j][e]; }
    }
  }
  __syncthreads();
  for (int c = threadIdx.x; c < NS * d; c += blockDim.x) {
    float acc = 0.f;
    for (int w = 0; w < groups_per_block; ++w) acc += sh[(size_t)w * NS * d + c];
    float* dst = c < d ? dgamma + c : c < 2 * d ? dbeta + (c - d) : c < 3 * d ? sum_dres + (c - 2 * d) : sum_dx + (c - 3 * d);
    if (c < 2 * d || (c < 3 * d ? sum_dres != nullptr : sum_dx != nullptr)) atomicAdd(dst, acc);
  }
}

// ------------------------------------------------------------------ BatchNorm1D  x:[batch, n]
// one thread per feature column; coalesced across threads for every row
template <typename T>
__global__ void batchnorm_fwd_kernel(const T* __restrict__ x, const float* __restrict__ gamma,
                                     const float* __restrict__ beta, T* __restrict__ y, float* __restrict__ mean_out,
                                     float* __restrict__ rstd_out, float* __restrict__ run_mean,
                                     float* __restrict__ run_var, int batch, int n, float eps, float momentum,
                                     int training) {
  int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= n) return;
  float mean, rstd;
  if (training) {
    float s = 0.f;
    for (int r = 0; r < batch; ++r) s += ldf(x + (long long)r * n + c);
    mean = s / batch;
    float q = 0.f;
    for (int r = 0; r < batch; ++r) { float a = ldf(x + (long long)r * n + c) - mean; q += a * a; }
    float var = q / batch;
    rstd = rsqrtf(var + eps);
    if (run_mean) {
      run_mean[c] = (1.f - momentum) * run_mean[c] + momentum * mean;
      float unb = batch > 1 ? var * batch / (batch - 1) : var;
      run_var[c] = (1.f - momentum) * run_var[c] + momentum * unb;
    }
  } else {
    mean = run_mean[c]; rstd = rsqrtf(run_var[c] + eps);
  }
  if (mean_out) { mean_out[c] = mean; rstd_out[c] = rstd; }
  const float g = gamma[c], b = beta[c];
  for (int r = 0; r < batch; ++r) {
    long long i = (long long)r * n + c;
    stf(y + i, (ldf(x + i) - mean) * rstd * g + b);
  }
}

template <typename T>
__global__ void batchnorm_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x, const float* __restrict__ gamma,
                                     const float* __restrict__ mean_in, const float* __restrict__ rstd_in,
                                     T* __restrict__ dx, float* __restrict__ dgamma, float* __restrict__ dbeta,
                                     int batch, int n, int training) {
  int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= n) return;
  const float mean = mean_in[c], rstd = rstd_in[c], g = gamma[c];
  float sg = 0.f, sgx = 0.f;
  for (int r = 0; r < batch; ++r) {
    long long i = (long long)r * n + c;
    float gy = ldf(dy + i); float xh = (ldf(x + i) - mean) * rstd;
    sg += gy; sgx += gy * xh;
  }
  dgamma[c] += sgx; dbeta[c] += sg;
  for (int r = 0; r < batch; ++r) {
    long long i = (long long)r * n + c;
    float gy = ldf(dy + i); float xh = (ldf(x + i) - mean) * rstd;
    float v = training ? g * rstd * (gy - sg / batch - xh * sgx / batch) : g * rstd * gy;
    stf(dx + i, v);
  }
}

}  // namespace b200

using namespace b200;

extern "C" {

static int layernorm_fwd_vec_dispatch(const void* x, const float* gamma, const float* beta, void* y, float* mean, float* rstd,
                                      long long rows, int d, float eps, const void* res, void* sum_out, cudaStream_t st);

// y = LayerNorm(x + res), sum_out = x + res (bf16 only, row width as the 16-byte-access kernel takes it; -1 otherwise)
int b200_add_layernorm_fwd(const void* x, const void* res, const float* gamma, const float* beta, void* sum_out, void* y, float* mean,
                           float* rstd, long long rows, int d, float eps, cudaStream_t st) {
  if (rows <= 0) return 0;
  if (((uintptr_t)res | (uintptr_t)sum_out) % 16) return -1;
  return layernorm_fwd_vec_dispatch(x, gamma, beta, y, mean, rstd, rows, d, eps, res, sum_out, st);
}

int b200_layernorm_fwd(const void* x, const float* gamma, const float* beta, void* y, float* mean, float* rstd,
                       long long rows, int d, float eps, int is_bf16, cudaStream_t st) {
  if (rows <= 0) return 0;
  const int block = 256, wpb = block / 32;
  long long g = (rows + wpb - 1) / wpb; if (g > 148 * 8) g = 148 * 8;
  if (is_bf16) {
    const int rc = layernorm_fwd_vec_dispatch(x, gamma, beta, y, mean, rstd, rows, d, eps, nullptr, nullptr, st);
    if (rc != -1) return rc;
  }
  if (is_bf16) layernorm_fwd_kernel<__nv_bfloat16><<<(int)g, block, 0, st>>>((const __nv_bfloat16*)x, gamma, beta, (__nv_bfloat16*)y, mean, rstd, rows, d, eps);
  else layernorm_fwd_kernel<float><<<(int)g, block, 0, st>>>((const float*)x, gamma, beta, (float*)y, mean, rstd, rows, d, eps);
  return (int)cudaGetLastError();
}


static int layernorm_fwd_vec_dispatch(const void* x, const float* gamma, const float* beta, void* y, float* mean, float* rstd,
                                      long long rows, int d, float eps, const void* res, void* sum_out, cudaStream_t st) {
  const int block = 256, wpb = block / 32;
  const bool fwd_vec_d = d % 256 == 0 && (d <= 1024 || d == 1536 || d == 2048 || d == 3072 || d == 4096);
  if (fwd_vec_d && (uintptr_t)x % 16 == 0 && (uintptr_t)y % 16 == 0 && (uintptr_t)gamma % 16 == 0 && (uintptr_t)beta % 16 == 0) {
#define B200_LNF(JJ, WW) { const int gpb = wpb / WW; long long gg = (rows + gpb - 1) / gpb; if (gg > 148 * 8) gg = 148 * 8; \
      launch_pdl(layernorm_fwd_vec_kernel<JJ, WW>, dim3((int)gg), dim3(block), 0, st, (const __nv_bfloat16*)x, gamma, beta, (__nv_bfloat16*)y, mean, rstd, rows, d, eps, (const __nv_bfloat16*)res, (__nv_bfloat16*)sum_out); }
    switch (d / 256) {
      case 1: B200_LNF(1, 1) break; case 2: B200_LNF(2, 1) break; case 3: B200_LNF(3, 1) break; case 4: B200_LNF(4, 1) break;
      case 6: B200_LNF(3, 2) break; case 8: B200_LNF(4, 2) break; case 12: B200_LNF(3, 4) break; default: B200_LNF(4, 4) break;
    }
#undef B200_LNF
    return (int)cudaGetLastError();
  }
  return -1;
}

// dgamma / dbeta are accumulated into (caller zero-initialises for a fresh gradient)
int b200_layernorm_bwd(const void* dy, const void* x, const float* gamma, const float* mean, const float* rstd,
                       void* dx, float* dgamma, float* dbeta, const void* dres, long long rows, int d, int is_bf16,
                       cudaStream_t st) {
  if (rows <= 0) return 0;
  const int block = 256, wpb = block / 32;
  long long g = (rows + wpb - 1) / wpb; if (g > 148 * 2) g = 148 * 2;
  const bool aligned16 = ((uintptr_t)dy % 16 == 0) && ((uintptr_t)x % 16 == 0) && ((uintptr_t)dx % 16 == 0) && (!dres || (uintptr_t)dres % 16 == 0) &&
                         ((uintptr_t)gamma % 16 == 0);
  const bool bwd_vec_d = d % 256 == 0 && (d <= 1024 || d == 1536 || d == 2048 || d == 3072 || d == 4096);
  if (is_bf16 && bwd_vec_d && aligned16) {
#define B200_LNV(JJ, WW) { auto k = layernorm_bwd_vec_kernel<JJ, WW>; const int gpb = wpb / WW; \
      const size_t sm = (size_t)gpb * 2 * d * sizeof(float); \
      long long gg = (rows + gpb - 1) / gpb; if (gg > 148 * 2) gg = 148 * 2; \
      if (sm + 256 > 48 * 1024) { cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm); if (e != cudaSuccess) return (int)e; } \
      launch_pdl(k, dim3((int)gg), dim3(block), sm, st, (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, gamma, (const float*)mean, (const float*)rstd, (__nv_bfloat16*)dx, dgamma, dbeta, (const __nv_bfloat16*)dres, rows, d, (float*)nullptr, (float*)nullptr); }
    switch (d / 256) {
      case 1: B200_LNV(1, 1) break; case 2: B200_LNV(2, 1) break; case 3: B200_LNV(3, 1) break; case 4: B200_LNV(4, 1) break;
      case 6: B200_LNV(3, 2) break; case 8: B200_LNV(4, 2) break; case 12: B200_LNV(3, 4) break; default: B200_LNV(4, 4) break;
    }
#undef B200_LNV
    return (int)cudaGetLastError();
  }
  if (d % 2 == 0 && d <= 1024) {
    const size_t sm = (size_t)wpb * 2 * d * sizeof(float);   // <= 64 KB
#define B200_LNB(TT, JJ) { auto k = layernorm_bwd_reg_kernel<TT, JJ>; \
      if (sm + 256 > 48 * 1024) { cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm); if (e != cudaSuccess) return (int)e; } \
      k<<<(int)g, block, sm, st>>>((const TT*)dy, (const TT*)x, gamma, mean, rstd, (TT*)dx, dgamma, dbeta, (const TT*)dres, rows, d); }
    if (is_bf16) { if (d <= 256) B200_LNB(__nv_bfloat16, 4) else if (d <= 512) B200_LNB(__nv_bfloat16, 8) else B200_LNB(__nv_bfloat16, 16) }
    else { if (d <= 256) B200_LNB(float, 4) else if (d <= 512) B200_LNB(float, 8) else B200_LNB(float, 16) }
#undef B200_LNB
    return (int)cudaGetLastError();
  }
  size_t smem = 2 * (size_t)d * sizeof(float);
  if (smem > 48 * 1024) {
    cudaError_t e;
    if (is_bf16) e = cudaFuncSetAttribute(layernorm_bwd_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    else e = cudaFuncSetAttribute(layernorm_bwd_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  if (is_bf16) layernorm_bwd_kernel<__nv_bfloat16><<<(int)g, block, smem, st>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, gamma, mean, rstd, (__nv_bfloat16*)dx, dgamma, dbeta, (const __nv_bfloat16*)dres, rows, d);
  else layernorm_bwd_kernel<float><<<(int)g, block, smem, st>>>((const float*)dy, (const float*)x, gamma, mean, rstd, (float*)dx, dgamma, dbeta, (const float*)dres, rows, d);
  return (int)cudaGetLastError();
}

// LayerNorm backward that also adds the column sums of `dres` and of dx (+ dres) into sum_dres / sum_dx (either may be
// null). bf16 rows with d a multiple of 256 up to 1024 and 16-byte aligned operands; returns -1 otherwise (the caller
// then takes b200_layernorm_bwd and separate column sums).
int b200_layernorm_bwd_sums(const void* dy, const void* x, const float* gamma, const float* mean, const float* rstd, void* dx,
                            float* dgamma, float* dbeta, const void* dres, long long rows, int d, float* sum_dres, float* sum_dx,
                            cudaStream_t st) {
  if (rows <= 0) return 0;
  const bool aligned16 = ((uintptr_t)dy % 16 == 0) && ((uintptr_t)x % 16 == 0) && ((uintptr_t)dx % 16 == 0) && (!dres || (uintptr_t)dres % 16 == 0) &&
                         ((uintptr_t)gamma % 16 == 0);
  if (!aligned16 || d % 256 != 0 || d > 1024) return -1;
  const int block = 256, gpb = block / 32;
  const size_t sm = (size_t)gpb * 4 * d * sizeof(float);
  long long gg = (rows + gpb - 1) / gpb; if (gg > 148 * 2) gg = 148 * 2;
#define B200_LNS(JJ) { auto k = layernorm_bwd_vec_kernel<JJ, 1, true>; \
    if (sm + 256 > 48 * 1024) { cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm); if (e != cudaSuccess) return (int)e; } \
    launch_pdl(k, dim3((int)gg), dim3(block), sm, st, (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, gamma, (const float*)mean, (const float*)rstd, (__nv_bfloat16*)dx, dgamma, dbeta, (const __nv_bfloat16*)dres, rows, d, sum_dres, sum_dx); }
  switch (d / 256) { case 1: B200_LNS(1) break; case 2: B200_LNS(2) break; case 3: B200_LNS(3) break; default: B200_LNS(4) break; }
#undef B200_LNS
  return (int)cudaGetLastError();
}

int b200_batchnorm_fwd(const void* x, const float* gamma, const float* beta, void* y, float* mean, float* rstd,
                       float* run_mean, float* run_var, int batch, int n, float eps, float momentum, int training,
                       int is_bf16, cudaStream_t st) {
  if (n <= 0 || batch <= 0) return 0;
  int grid = (n + 127) / 128;
  if (is_bf16) batchnorm_fwd_kernel<__nv_bfloat16><<<grid, 128, 0, st>>>((const __nv_bfloat16*)x, gamma, beta, (__nv_bfloat16*)y, mean, rstd, run_mean, run_var, batch, n, eps, momentum, training);
  else batchnorm_fwd_kernel<float><<<grid, 128, 0, st>>>((const float*)x, gamma, beta, (float*)y, mean, rstd, run_mean, run_var, batch, n, eps, momentum, training);
  return (int)cudaGetLastError();
}

int b200_batchnorm_bwd(const void* dy, const void* x, const float* gamma, const float* mean, const float* rstd,
                       void* dx, float* dgamma, float* dbeta, int batch, int n, int training, int is_bf16,
                       cudaStream_t st) {
  if (n <= 0 || batch <= 0) return 0;
  int grid = (n + 127) / 128;
  if (is_bf16) batchnorm_bwd_kernel<__nv_bfloat16><<<grid, 128, 0, st>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, gamma, mean, rstd, (__nv_bfloat16*)dx, dgamma, dbeta, batch, n, training);
  else batchnorm_bwd_kernel<float><<<grid, 128, 0, st>>>((const float*)dy, (const float*)x, gamma, mean, rstd, (float*)dx, dgamma, dbeta, batch, n, training);
  return (int)cudaGetLastError();
}

}  // extern "C"
