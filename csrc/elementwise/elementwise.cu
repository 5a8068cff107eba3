// E1: vectorised elementwise / broadcast / reduce family (HBM-bound; 16-byte accesses, grid-stride).
// Restates the reference's AVX2 elementwise helpers (rust-nn src/simd.rs:214-406), its activation
// shader (src/gpu.rs:136-153), Dropout (src/nn.rs:231-259), FakeQuantize (src/nn.rs:644-667),
// softplus/sigmoid/silu ops (src/tensor.rs:948-987) and the bias column-sum of the Linear backward
// (src/tensor.rs:1592-1709) as CUDA kernels.
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cstdint>
#include "../gemm/gemm_sm100.h"
#include "../common/launch.cuh"

namespace b200 {

template <typename T> struct Vec;
template <> struct Vec<float> { using V = float4; static constexpr int N = 4; };
template <> struct Vec<__nv_bfloat16> { using V = uint4; static constexpr int N = 8; };

template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16(v); }

template <typename T, int N> struct alignas(sizeof(T) * N) Pack { T v[N]; };

__device__ __forceinline__ float gelu_f(float v) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  return 0.5f * v * (1.f + tanhf(k0 * (v + k1 * v * v * v)));
}
__device__ __forceinline__ float gelu_grad(float s) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  float t = tanhf(k0 * (s + k1 * s * s * s));
  return 0.5f * (1.f + t) + 0.5f * s * (1.f - t * t) * k0 * (1.f + 3.f * k1 * s * s);
}
__device__ __forceinline__ float softplus_f(float v) { return v > 20.f ? v : log1pf(__expf(v)); }

enum : int {
  OP_ADD = 0, OP_SUB = 1, OP_MUL = 2, OP_DIV = 3,
  OP_RELU = 10, OP_GELU = 11, OP_SILU = 12, OP_SIGMOID = 13, OP_TANH = 14, OP_SOFTPLUS = 15,
  OP_SCALE = 16, OP_EXP = 17, OP_ABS = 18, OP_SQUARE = 19, OP_CLAMP = 20, OP_ROUND = 21, OP_ADD_SCALAR = 22,
  // linear-attention feature maps of (s0 * x): elu(x)+1 and relu(x)^2 (rust-nn src/linear_attention.rs:42-94)
  OP_ELU1 = 23, OP_RELU2 = 24,
  // backward of a unary op: out = g * f'(saved); saved is the INPUT of the forward op
  OP_RELU_BWD = 30, OP_GELU_BWD = 31, OP_SILU_BWD = 32, OP_SIGMOID_BWD = 33, OP_TANH_BWD = 34, OP_SOFTPLUS_BWD = 35,
  // fused: out = a * silu(b)  (Mamba gate) and its two gradients
  OP_SIGMOID_BWD_OUT = 36, OP_TANH_BWD_OUT = 37,
  OP_DIV_BWD_B = 38,   // -a * b
  OP_ELU1_BWD = 41, OP_RELU2_BWD = 42,   // saved = the (already scaled) input of the feature map
  OP_MUL_SILU = 40,
};

__device__ __forceinline__ float unary_apply(float x, int op, float s0, float s1) {
  switch (op) {
    case OP_RELU: return x > 0.f ? x : 0.f;
    case OP_GELU: return gelu_f(x);
    case OP_SILU: return x / (1.f + __expf(-x));
    case OP_SIGMOID: return 1.f / (1.f + __expf(-x));
    case OP_TANH: return tanhf(x);
    case OP_SOFTPLUS: return softplus_f(x);
    case OP_SCALE: return x * s0;
    case OP_ADD_SCALAR: return x + s0;
    case OP_EXP: return __expf(x);
    case OP_ABS: return fabsf(x);
    case OP_SQUARE: return x * x;
    case OP_CLAMP: return fminf(fmaxf(x, s0), s1);
    case OP_ROUND: return rintf(x);
    case OP_ELU1: { float v = x * s0; return v > 0.f ? v + 1.f : __expf(v); }
    case OP_RELU2: { float v = x * s0; return v > 0.f ? v * v : 0.f; }
    default: return x;
  }
}
__device__ __forceinline__ float binary_apply(float a, float b, int op) {
  switch (op) {
    case OP_ADD: return a + b;
    case OP_SUB: return a - b;
    case OP_MUL: return a * b;
    case OP_DIV: return a / b;
    case OP_RELU_BWD: return b > 0.f ? a : 0.f;
    case OP_GELU_BWD: return a * gelu_grad(b);
    case OP_SILU_BWD: { float sg = 1.f / (1.f + __expf(-b)); return a * sg * (1.f + b * (1.f - sg)); }
    case OP_SIGMOID_BWD: { float sg = 1.f / (1.f + __expf(-b)); return a * sg * (1.f - sg); }
    case OP_TANH_BWD: { float t = tanhf(b); return a * (1.f - t * t); }
    case OP_SOFTPLUS_BWD: return a / (1.f + __expf(-b));
    case OP_SIGMOID_BWD_OUT: return a * b * (1.f - b);
    case OP_TANH_BWD_OUT: return a * (1.f - b * b);
    case OP_DIV_BWD_B: return -a * b;
    case OP_ELU1_BWD: return b > 0.f ? a : a * __expf(b);
    case OP_RELU2_BWD: return b > 0.f ? 2.f * a * b : 0.f;
    case OP_MUL_SILU: return a * b / (1.f + __expf(-b));
    default: return a;
  }
}

template <typename T>
__global__ void unary_kernel(const T* __restrict__ x, T* __restrict__ y, long long n, int op, float s0, float s1) {
  constexpr int N = Vec<T>::N;
  using P = Pack<T, N>;
  long long nv = n / N;
  long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  long long stride = (long long)gridDim.x * blockDim.x;
  for (; i < nv; i += stride) {
    P in = reinterpret_cast<const P*>(x)[i], out;
#pragma unroll
    for (int j = 0; j < N; ++j) out.v[j] = from_f<T>(unary_apply(to_f(in.v[j]), op, s0, s1));
    reinterpret_cast<P*>(y)[i] = out;
  }
  long long tail = nv * N + blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (tail < n) y[tail] = from_f<T>(unary_apply(to_f(x[tail]), op, s0, s1));
}

// y = a (op) b with b broadcast along rows when b_period > 0 (b has b_period elements, index = i % b_period)
template <typename T>
__global__ void binary_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ y, long long n,
                              int op, long long b_period) {
  pdl_trigger();
  pdl_wait();
  constexpr int N = Vec<T>::N;
  using P = Pack<T, N>;
  long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  long long stride = (long long)gridDim.x * blockDim.x;
  if (b_period == 0) {
    long long nv = n / N;
    for (long long k = i; k < nv; k += stride) {
      P pa = reinterpret_cast<const P*>(a)[k], pb = reinterpret_cast<const P*>(b)[k], out;
#pragma unroll
      for (int j = 0; j < N; ++j) out.v[j] = from_f<T>(binary_apply(to_f(pa.v[j]), to_f(pb.v[j]), op));
      reinterpret_cast<P*>(y)[k] = out;
    }
    long long tail = nv * N + i;
    if (tail < n) y[tail] = from_f<T>(binary_apply(to_f(a[tail]), to_f(b[tail]), op));
  } else if (b_period % N == 0 && n % N == 0) {
    long long nv = n / N;
    for (long long k = i; k < nv; k += stride) {
      P pa = reinterpret_cast<const P*>(a)[k], pb = reinterpret_cast<const P*>(b)[(k * N % b_period) / N], out;
#pragma unroll
      for (int j = 0; j < N; ++j) out.v[j] = from_f<T>(binary_apply(to_f(pa.v[j]), to_f(pb.v[j]), op));
      reinterpret_cast<P*>(y)[k] = out;
    }
  } else {
    for (long long k = i; k < n; k += stride)
      y[k] = from_f<T>(binary_apply(to_f(a[k]), to_f(b[k % b_period]), op));
  }
}

// Mamba output gate on row-strided bf16 matrices (the gate z is a column slice of the fused input projection's output,
// so its rows are 2 x cols apart): out = y * silu(z), and its backward in one pass over g, y, z:
// dy = g * silu(z), dz = g * y * silu'(z). 16-byte packets, four per thread in flight.
__device__ __forceinline__ void gate_unpack(const uint4& u, float (&f)[8]) {
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int k = 0; k < 4; ++k) { f[2 * k] = __uint_as_float(w[k] << 16); f[2 * k + 1] = __uint_as_float(w[k] & 0xffff0000u); }
}
__device__ __forceinline__ uint4 gate_pack(const float (&f)[8]) {
  uint32_t w[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) { const __nv_bfloat162 t = __floats2bfloat162_rn(f[2 * k], f[2 * k + 1]); w[k] = *reinterpret_cast<const uint32_t*>(&t); }
  return make_uint4(w[0], w[1], w[2], w[3]);
}
template <bool BWD>
__global__ void __launch_bounds__(256)
gate_kernel(const __nv_bfloat16* __restrict__ g, long long ld_g, const __nv_bfloat16* __restrict__ y, long long ld_y,
            const __nv_bfloat16* __restrict__ z, long long ld_z, __nv_bfloat16* __restrict__ o0, long long ld_0,
            __nv_bfloat16* __restrict__ o1, long long ld_1, unsigned rows, unsigned ppr) {
  pdl_trigger();
  pdl_wait();
  const unsigned total = rows * ppr, stride = gridDim.x * blockDim.x;
  for (unsigned k0 = blockIdx.x * blockDim.x + threadIdx.x; k0 < total; k0 += 4 * stride) {
    uint4 a[4], b[4], c[4];
    long long r[4]; unsigned col[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const unsigned k = k0 + u * stride;
      r[u] = k / ppr; col[u] = (k - (unsigned)r[u] * ppr) * 8;
      if (k < total) {
        b[u] = __ldg(reinterpret_cast<const uint4*>(y + r[u] * ld_y + col[u]));
        c[u] = __ldg(reinterpret_cast<const uint4*>(z + r[u] * ld_z + col[u]));
        if (BWD) a[u] = __ldg(reinterpret_cast<const uint4*>(g + r[u] * ld_g + col[u]));
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      if (k0 + u * stride >= total) continue;
      float fy[8], fz[8], r0[8], r1[8];
      gate_unpack(b[u], fy); gate_unpack(c[u], fz);
      if (BWD) {
        float fg[8];
        gate_unpack(a[u], fg);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float sg = __fdividef(1.f, 1.f + __expf(-fz[e])), sl = fz[e] * sg;
          r0[e] = fg[e] * sl;                                              // d y
          r1[e] = fg[e] * fy[e] * sg * (1.f + fz[e] * (1.f - sg));          // d z
        }
        *reinterpret_cast<uint4*>(o0 + r[u] * ld_0 + col[u]) = gate_pack(r0);
        *reinterpret_cast<uint4*>(o1 + r[u] * ld_1 + col[u]) = gate_pack(r1);
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) r0[e] = fy[e] * fz[e] * __fdividef(1.f, 1.f + __expf(-fz[e]));
        *reinterpret_cast<uint4*>(o0 + r[u] * ld_0 + col[u]) = gate_pack(r0);
      }
    }
  }
}

// cast kernels
template <typename TI, typename TO>
__global__ void cast_kernel(const TI* __restrict__ x, TO* __restrict__ y, long long n, float scale) {
  long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  long long stride = (long long)gridDim.x * blockDim.x;
  for (; i < n; i += stride) y[i] = from_f<TO>(to_f(x[i]) * scale);
}

// column sum: out[c] (+)= sum_r x[r, c]   (dbias). Two-stage: each block reduces a slab of rows, atomics to fp32.
template <typename T>
__global__ void colsum_kernel(const T* __restrict__ x, float* __restrict__ out, long long rows, int cols,
                              long long ld, int rows_per_block) {
  int c = blockIdx.x * blockDim.x + threadIdx.x;
  long long r0 = (long long)blockIdx.y * rows_per_block;
  long long r1 = r0 + rows_per_block; if (r1 > rows) r1 = rows;
  if (c >= cols) return;
  float acc = 0.f;
  for (long long r = r0; r < r1; ++r) acc += to_f(x[r * ld + c]);
  atomicAdd(out + c, acc);
}

// bf16 column sum with 16-byte loads: a warp covers 256 columns of one row per load, the block's 8 warps
// take rows w, w + 8, ... of the block's slab (4 rows in flight per lane), then the warps' partial sums meet in
// shared memory and leave as one atomic per column. Needs cols % 8 == 0, ld % 8 == 0 and a 16-byte aligned base.
__global__ void __launch_bounds__(256)
colsum_vec_kernel(const __nv_bfloat16* __restrict__ x, float* __restrict__ out, long long rows, int cols, long long ld, int rows_per_block) {
  __shared__ float sh[8][256 + 8];
  pdl_trigger();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int c0 = blockIdx.x * 256 + lane * 8;
  const long long r0 = (long long)blockIdx.y * rows_per_block;
  long long r1 = r0 + rows_per_block; if (r1 > rows) r1 = rows;
  float acc[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) acc[k] = 0.f;
  if (c0 < cols) {
    const __nv_bfloat16* xp = x + c0;
    long long r = r0 + warp;
    for (; r + 24 < r1; r += 32) {
      uint4 v[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) v[j] = __ldg(reinterpret_cast<const uint4*>(xp + (r + 8 * j) * ld));
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint32_t w[4] = {v[j].x, v[j].y, v[j].z, v[j].w};
#pragma unroll
        for (int k = 0; k < 4; ++k) { acc[2 * k] += __uint_as_float(w[k] << 16); acc[2 * k + 1] += __uint_as_float(w[k] & 0xffff0000u); }
      }
    }
    for (; r < r1; r += 8) {
      const uint4 v = __ldg(reinterpret_cast<const uint4*>(xp + r * ld));
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) { acc[2 * k] += __uint_as_float(w[k] << 16); acc[2 * k + 1] += __uint_as_float(w[k] & 0xffff0000u); }
    }
  }
#pragma unroll
  for (int k = 0; k < 8; ++k) sh[warp][lane * 8 + k] = acc[k];
  __syncthreads();
  const int c = blockIdx.x * 256 + threadIdx.x;
  if (c < cols) {
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) t += sh[w][threadIdx.x];
    atomicAdd(out + c, t);
  }
}

// Activation backward + bias gradient in one pass: g[r, c] *= act'(saved[r, c]) in place and dbias[c] += the column
// sums of the result. A GEMM epilogue that reads `saved` is latency-bound (each epilogue warp has 4 KB outstanding);
// as a streaming kernel the same work runs at copy bandwidth, and the column sum costs no extra pass.
// Same thread layout as colsum_vec_kernel. OP is OP_GELU_BWD / OP_SILU_BWD / OP_RELU_BWD; the derivatives use the
// hardware tanh / exp approximations (relative error ~2^-11, below the bf16 result's own rounding).
template <int OP>
__device__ __forceinline__ float dact_fast(float a, float s) {
  if constexpr (OP == OP_RELU_BWD) return s > 0.f ? a : 0.f;
  else if constexpr (OP == OP_GELU_BWD) {
    const float k0 = 0.7978845608028654f, k1 = 0.044715f;
    float t;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(k0 * (s + k1 * s * s * s)));
    return a * (0.5f * (1.f + t) + 0.5f * s * (1.f - t * t) * (k0 * (1.f + 3.f * k1 * s * s)));
  } else {
    const float sg = __fdividef(1.f, 1.f + __expf(-s));
    return a * sg * (1.f + s * (1.f - sg));
  }
}
template <int OP>
__global__ void __launch_bounds__(256)
dact_colsum_kernel(__nv_bfloat16* __restrict__ g, const __nv_bfloat16* __restrict__ saved, float* __restrict__ dbias, long long rows, int cols,
                   long long ld_g, long long ld_s, int rows_per_block) {
  __shared__ float sh[8][256 + 8];
  pdl_trigger();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int c0 = blockIdx.x * 256 + lane * 8;
  const long long r0 = (long long)blockIdx.y * rows_per_block;
  long long r1 = r0 + rows_per_block; if (r1 > rows) r1 = rows;
  float acc[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) acc[k] = 0.f;
  if (c0 < cols) {
    auto one = [&](uint4& gv, const uint4& sv) {
      uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w};
      const uint32_t sw[4] = {sv.x, sv.y, sv.z, sv.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float lo = dact_fast<OP>(__uint_as_float(gw[k] << 16), __uint_as_float(sw[k] << 16));
        const float hi = dact_fast<OP>(__uint_as_float(gw[k] & 0xffff0000u), __uint_as_float(sw[k] & 0xffff0000u));
        const __nv_bfloat162 pk = __floats2bfloat162_rn(lo, hi);
        gw[k] = *reinterpret_cast<const uint32_t*>(&pk);
        acc[2 * k] += __low2float(pk); acc[2 * k + 1] += __high2float(pk);       // sums of the ROUNDED values, as a later colsum would see
      }
      gv = make_uint4(gw[0], gw[1], gw[2], gw[3]);
    };
    long long r = r0 + warp;
    for (; r + 24 < r1; r += 32) {                   // four rows of both operands in flight per lane
      uint4 gv[4], sv[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        gv[j] = *reinterpret_cast<const uint4*>(g + (r + 8 * j) * ld_g + c0);
        sv[j] = __ldg(reinterpret_cast<const uint4*>(saved + (r + 8 * j) * ld_s + c0));
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        one(gv[j], sv[j]);
        *reinterpret_cast<uint4*>(g + (r + 8 * j) * ld_g + c0) = gv[j];
      }
    }
    for (; r + 8 < r1; r += 16) {
      uint4 gv[2], sv[2];
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        gv[j] = *reinterpret_cast<const uint4*>(g + (r + 8 * j) * ld_g + c0);
        sv[j] = __ldg(reinterpret_cast<const uint4*>(saved + (r + 8 * j) * ld_s + c0));
      }
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        one(gv[j], sv[j]);
        *reinterpret_cast<uint4*>(g + (r + 8 * j) * ld_g + c0) = gv[j];
      }
    }
    for (; r < r1; r += 8) {
      uint4 gv = *reinterpret_cast<const uint4*>(g + r * ld_g + c0);
      const uint4 sv = __ldg(reinterpret_cast<const uint4*>(saved + r * ld_s + c0));
      one(gv, sv);
      *reinterpret_cast<uint4*>(g + r * ld_g + c0) = gv;
    }
  }
  if (dbias == nullptr) return;
#pragma unroll
  for (int k = 0; k < 8; ++k) sh[warp][lane * 8 + k] = acc[k];
  __syncthreads();
  const int c = blockIdx.x * 256 + threadIdx.x;
  if (c < cols) {
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) t += sh[w][threadIdx.x];
    atomicAdd(dbias + c, t);
  }
}

// batched column sum: out[z, c] += sum_r x[z, r, c]  (per-expert bias gradients)
template <typename T>
__global__ void colsum_batched_kernel(const T* __restrict__ x, float* __restrict__ out, long long rows, int cols,
                                      long long ld, long long bs, const int* __restrict__ rows_valid) {
  int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  const T* xp = x + blockIdx.z * bs;
  if (rows_valid) { const long long rv = ((long long)rows_valid[blockIdx.z] + 127) / 128 * 128; if (rv < rows) rows = rv; }   // ragged groups: whole 128-row tiles
  long long r0 = (long long)blockIdx.y * 256, r1 = r0 + 256; if (r1 > rows) r1 = rows;
  if (r0 >= r1) return;
  float acc = 0.f;
  for (long long r = r0; r < r1; ++r) acc += to_f(xp[r * ld + c]);
  atomicAdd(out + (long long)blockIdx.z * cols + c, acc);
}

// full reduction sum / sum of squares / max / min into fp32 scalar slots (out[0..3])
template <typename T>
__global__ void reduce_kernel(const T* __restrict__ x, float* __restrict__ out, long long n, int what) {
  float acc = (what == 2) ? -INFINITY : (what == 3) ? INFINITY : 0.f;
  long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  long long stride = (long long)gridDim.x * blockDim.x;
  for (; i < n; i += stride) {
    float v = to_f(x[i]);
    if (what == 0) acc += v; else if (what == 1) acc += v * v; else if (what == 2) acc = fmaxf(acc, v); else acc = fminf(acc, v);
  }
  __shared__ float sh[32];
  for (int o = 16; o > 0; o >>= 1) {
    float t = __shfl_xor_sync(0xffffffffu, acc, o);
    if (what <= 1) acc += t; else if (what == 2) acc = fmaxf(acc, t); else acc = fminf(acc, t);
  }
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    int nw = blockDim.x >> 5;
    acc = threadIdx.x < nw ? sh[threadIdx.x] : ((what == 2) ? -INFINITY : (what == 3) ? INFINITY : 0.f);
    for (int o = 16; o > 0; o >>= 1) {
      float t = __shfl_xor_sync(0xffffffffu, acc, o);
      if (what <= 1) acc += t; else if (what == 2) acc = fmaxf(acc, t); else acc = fminf(acc, t);
    }
    if (threadIdx.x == 0) {
      if (what <= 1) atomicAdd(out, acc);
      else if (what == 2) { int* a = (int*)out; int old = *a, assumed; do { assumed = old; if (__int_as_float(assumed) >= acc) break; old = atomicCAS(a, assumed, __float_as_int(acc)); } while (assumed != old); }
      else { int* a = (int*)out; int old = *a, assumed; do { assumed = old; if (__int_as_float(assumed) <= acc) break; old = atomicCAS(a, assumed, __float_as_int(acc)); } while (assumed != old); }
    }
  }
}

// Philox-free counter hash (splitmix64) for dropout: stateless, seed + element index.
__device__ __forceinline__ float u01(uint64_t seed, uint64_t idx) {
  uint64_t z = seed + idx * 0x9E3779B97F4A7C15ull + 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  z = z ^ (z >> 31);
  return (float)(z >> 40) * (1.0f / 16777216.0f);
}
template <typename T>
__global__ void dropout_kernel(const T* __restrict__ x, T* __restrict__ y, long long n, float p, float scale,
                               uint64_t seed) {
  long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  long long stride = (long long)gridDim.x * blockDim.x;
  for (; i < n; i += stride) {
    float keep = u01(seed, (uint64_t)i) >= p ? scale : 0.f;
    y[i] = from_f<T>(to_f(x[i]) * keep);
  }
}

// fake quantise: y = clamp(round(x / s), qmin, qmax) * s   (gradient is a straight-through mask, computed in python)
template <typename T>
__global__ void fake_quant_kernel(const T* __restrict__ x, T* __restrict__ y, long long n, float scale, float qmin,
                                  float qmax) {
  long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  long long stride = (long long)gridDim.x * blockDim.x;
  for (; i < n; i += stride) {
    float q = rintf(to_f(x[i]) / scale);
    q = fminf(fmaxf(q, qmin), qmax);
    y[i] = from_f<T>(q * scale);
  }
}

// embedding gather: out[t, :] = table[ids[t], :]  (bf16 or f32 rows, 16-byte vector copies)
template <typename T>
__global__ void embedding_fwd_kernel(const T* __restrict__ table, const long long* __restrict__ ids,
                                     T* __restrict__ out, long long tokens, int dim, long long vocab) {
  constexpr int N = Vec<T>::N;
  using P = Pack<T, N>;
  int vec_per_row = dim / N;
  long long total = tokens * vec_per_row;
  long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  long long stride = (long long)gridDim.x * blockDim.x;
  for (; i < total; i += stride) {
    long long t = i / vec_per_row; int v = (int)(i % vec_per_row);
    long long id = ids[t];
    if (id < 0 || id >= vocab) id = 0;
    reinterpret_cast<P*>(out + t * dim)[v] = reinterpret_cast<const P*>(table + id * dim)[v];
  }
}
// embedding backward: grad_table[ids[t], :] += g[t, :]  (fp32 accumulation)
template <typename T>
__global__ void embedding_bwd_kernel(const T* __restrict__ g, const long long* __restrict__ ids,
                                     float* __restrict__ grad_table, long long tokens, int dim, long long vocab) {
  long long total = tokens * dim;
  long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  long long stride = (long long)gridDim.x * blockDim.x;
  for (; i < total; i += stride) {
    long long t = i / dim; int d = (int)(i % dim);
    long long id = ids[t];
    if (id < 0 || id >= vocab) continue;
    atomicAdd(grad_table + id * dim + d, to_f(g[i]));
  }
}

// out[c, r] = in[r, c] for a batch of row-major matrices (32x32 tiles through shared memory)
template <typename T>
__global__ void transpose_kernel(const T* __restrict__ in, T* __restrict__ out, int rows, int cols, long long ld_in,
                                 long long ld_out, long long bs_in, long long bs_out) {
  __shared__ T tile[32][33];
  const T* src = in + blockIdx.z * bs_in; T* dst = out + blockIdx.z * bs_out;
  int c = blockIdx.x * 32 + threadIdx.x;
  for (int j = threadIdx.y; j < 32; j += blockDim.y) {
    int r = blockIdx.y * 32 + j;
    if (r < rows && c < cols) tile[j][threadIdx.x] = src[(long long)r * ld_in + c];
  }
  __syncthreads();
  int r2 = blockIdx.y * 32 + threadIdx.x;
  for (int j = threadIdx.y; j < 32; j += blockDim.y) {
    int c2 = blockIdx.x * 32 + j;
    if (r2 < rows && c2 < cols) dst[(long long)c2 * ld_out + r2] = tile[threadIdx.x][j];
  }
}

// P1 rotary embedding, rotate-half convention with duplicated-half tables [seq, dim]
// (rust-nn src/tensor.rs:1077-1124): out[i] = x[i] cos[i] - x[h+i] sin[i]; out[h+i] = x[h+i] cos[h+i] + x[i] sin[h+i].
// `sign` = -1 applies the inverse rotation, which is the backward pass (src/tensor.rs:2002-2013).
template <typename T>
__global__ void rope_kernel(const T* __restrict__ x, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                            T* __restrict__ y, long long leading, int seq, int dim, float sign) {
  const int half = dim / 2;
  const long long total = leading * seq * half;
  long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (; i < total; i += stride) {
    const int j = (int)(i % half); long long r = i / half;
    const int s = (int)(r % seq);
    const long long base = r * dim;
    const float xi = to_f(x[base + j]), xj = to_f(x[base + half + j]);
    const float c0 = cos_t[s * dim + j], c1 = cos_t[s * dim + half + j];
    const float s0 = sign * sin_t[s * dim + j], s1 = sign * sin_t[s * dim + half + j];
    y[base + j] = from_f<T>(xi * c0 - xj * s0);
    y[base + half + j] = from_f<T>(xj * c1 + xi * s1);
  }
}

static inline int grid_for(long long work, int block, int max_blocks = 148 * 16) {
  long long g = (work + block - 1) / block;
  if (g < 1) g = 1;
  if (g > max_blocks) g = max_blocks;
  return (int)g;
}


// Row softmax over the last axis (rust-nn src/activations.rs:23-62 is forward-only; here it has a backward). One block
// per row; the row is read twice (maximum + sum, then normalise), fp32 arithmetic. `scale` multiplies the input first;
// `causal_period` > 0 masks column j of row r when j > r % causal_period (rows of [.., S, S] score matrices).
template <typename T>
__global__ void softmax_fwd_kernel(const T* __restrict__ x, T* __restrict__ y, int cols, float scale, int causal_period) {
  const long long r = blockIdx.x;
  const T* xr = x + r * cols; T* yr = y + r * cols;
  const int limit = causal_period > 0 ? min(cols, (int)(r % causal_period) + 1) : cols;
  __shared__ float sh[33];
  float m = -INFINITY;
  for (int j = threadIdx.x; j < limit; j += blockDim.x) m = fmaxf(m, to_f(xr[j]) * scale);
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < (blockDim.x >> 5) ? sh[threadIdx.x] : -INFINITY;
    for (int o = 16; o > 0; o >>= 1) t = fmaxf(t, __shfl_xor_sync(0xffffffffu, t, o));
    if (threadIdx.x == 0) sh[32] = t;
  }
  __syncthreads();
  m = sh[32];
  __syncthreads();
  float sum = 0.f;
  for (int j = threadIdx.x; j < limit; j += blockDim.x) sum += __expf(to_f(xr[j]) * scale - m);
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = sum;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < (blockDim.x >> 5) ? sh[threadIdx.x] : 0.f;
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (threadIdx.x == 0) sh[32] = t;
  }
  __syncthreads();
  const float inv = 1.f / sh[32];
  for (int j = threadIdx.x; j < cols; j += blockDim.x) yr[j] = from_f<T>(j < limit ? __expf(to_f(xr[j]) * scale - m) * inv : 0.f);
}
// dx = scale * y * (dy - sum_j dy_j y_j)
template <typename T>
__global__ void softmax_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ y, T* __restrict__ dx, int cols, float scale) {
  const long long r = blockIdx.x;
  const T* gr = dy + r * cols; const T* yr = y + r * cols; T* dr = dx + r * cols;
  __shared__ float sh[33];
  float dot = 0.f;
  for (int j = threadIdx.x; j < cols; j += blockDim.x) dot += to_f(gr[j]) * to_f(yr[j]);
  for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = dot;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < (blockDim.x >> 5) ? sh[threadIdx.x] : 0.f;
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (threadIdx.x == 0) sh[32] = t;
  }
  __syncthreads();
  dot = sh[32];
  for (int j = threadIdx.x; j < cols; j += blockDim.x) dr[j] = from_f<T>(scale * to_f(yr[j]) * (to_f(gr[j]) - dot));
}

}  // namespace b200

using namespace b200;

extern "C" {

int b200_unary(const void* x, void* y, long long n, int op, float s0, float s1, int is_bf16, cudaStream_t st) {
  if (n <= 0) return 0;
  if (is_bf16) unary_kernel<__nv_bfloat16><<<grid_for(n / 8 + 1, 256), 256, 0, st>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y, n, op, s0, s1);
  else unary_kernel<float><<<grid_for(n / 4 + 1, 256), 256, 0, st>>>((const float*)x, (float*)y, n, op, s0, s1);
  return (int)cudaGetLastError();
}

int b200_binary(const void* a, const void* b, void* y, long long n, int op, long long b_period, int is_bf16,
                cudaStream_t st) {
  if (n <= 0) return 0;
  const int vw = is_bf16 ? 8 : 4;
  long long work = (b_period && (b_period % vw || n % vw)) ? n : n / vw + 1;
  if (is_bf16) launch_pdl(binary_kernel<__nv_bfloat16>, dim3(grid_for(work, 256)), dim3(256), 0, st, (const __nv_bfloat16*)a, (const __nv_bfloat16*)b, (__nv_bfloat16*)y, n, op, b_period);
  else launch_pdl(binary_kernel<float>, dim3(grid_for(work, 256)), dim3(256), 0, st, (const float*)a, (const float*)b, (float*)y, n, op, b_period);
  return (int)cudaGetLastError();
}

// Gate forward (g == nullptr: o0 = y * silu(z)) or backward (o0 = d y, o1 = d z). bf16, cols % 8 == 0, every leading
// dimension % 8 == 0, 16-byte aligned bases, fewer than 2^31 packets; -1 otherwise (the caller composes elementwise kernels).
int b200_gate(const void* g, long long ld_g, const void* y, long long ld_y, const void* z, long long ld_z, void* o0, long long ld_0,
              void* o1, long long ld_1, long long rows, int cols, cudaStream_t st) {
  if (rows <= 0 || cols <= 0) return 0;
  const bool bwd = g != nullptr;
  if (cols % 8 || ld_y % 8 || ld_z % 8 || ld_0 % 8 || (bwd && (ld_g % 8 || ld_1 % 8))) return -1;
  if (((uintptr_t)y | (uintptr_t)z | (uintptr_t)o0 | (uintptr_t)g | (uintptr_t)o1) & 15) return -1;
  const long long packets = rows * (cols / 8);
  if (packets >= (1LL << 31) - 4LL * 148 * 16 * 256) return -1;
  const dim3 grid(grid_for((packets + 3) / 4, 256));
  const __nv_bfloat16 *gp = (const __nv_bfloat16*)g, *yp = (const __nv_bfloat16*)y, *zp = (const __nv_bfloat16*)z;
  if (bwd) launch_pdl(gate_kernel<true>, grid, dim3(256), 0, st, gp, ld_g, yp, ld_y, zp, ld_z, (__nv_bfloat16*)o0, ld_0, (__nv_bfloat16*)o1, ld_1, (unsigned)rows, (unsigned)(cols / 8));
  else launch_pdl(gate_kernel<false>, grid, dim3(256), 0, st, gp, ld_g, yp, ld_y, zp, ld_z, (__nv_bfloat16*)o0, ld_0, (__nv_bfloat16*)o1, ld_1, (unsigned)rows, (unsigned)(cols / 8));
  return (int)cudaGetLastError();
}

// dir: 0 f32->bf16, 1 bf16->f32
int b200_cast(const void* x, void* y, long long n, float scale, int dir, cudaStream_t st) {
  if (n <= 0) return 0;
  if (dir == 0) cast_kernel<float, __nv_bfloat16><<<grid_for(n, 256), 256, 0, st>>>((const float*)x, (__nv_bfloat16*)y, n, scale);
  else cast_kernel<__nv_bfloat16, float><<<grid_for(n, 256), 256, 0, st>>>((const __nv_bfloat16*)x, (float*)y, n, scale);
  return (int)cudaGetLastError();
}

// g (bf16, in place) *= act'(saved); dbias (fp32, may be null) += column sums. Needs cols % 8 == 0, both leading
// dimensions % 8 == 0, 16-byte aligned bases and op in {relu, gelu, silu}_bwd (returns -1 otherwise: the caller falls
// back to two kernels).
int b200_dact_colsum(void* g, const void* saved, float* dbias, long long rows, int cols, long long ld_g, long long ld_s, int op, cudaStream_t st) {
  if (rows <= 0 || cols <= 0) return 0;
  if (cols % 8 || ld_g % 8 || ld_s % 8 || ((uintptr_t)g & 15) || ((uintptr_t)saved & 15)) return -1;
  const int cb = (cols + 255) / 256;
  long long rpb = (rows * cb + 148LL * 8 - 1) / (148LL * 8);
  rpb = rpb < 16 ? 16 : rpb > 512 ? 512 : (rpb + 15) / 16 * 16;
  dim3 grid(cb, (unsigned)((rows + rpb - 1) / rpb));
  __nv_bfloat16* gp = (__nv_bfloat16*)g;
  const __nv_bfloat16* sp = (const __nv_bfloat16*)saved;
  if (op == OP_GELU_BWD) launch_pdl(dact_colsum_kernel<OP_GELU_BWD>, grid, dim3(256), 0, st, gp, sp, dbias, rows, cols, ld_g, ld_s, (int)rpb);
  else if (op == OP_SILU_BWD) launch_pdl(dact_colsum_kernel<OP_SILU_BWD>, grid, dim3(256), 0, st, gp, sp, dbias, rows, cols, ld_g, ld_s, (int)rpb);
  else if (op == OP_RELU_BWD) launch_pdl(dact_colsum_kernel<OP_RELU_BWD>, grid, dim3(256), 0, st, gp, sp, dbias, rows, cols, ld_g, ld_s, (int)rpb);
  else return -1;
  return (int)cudaGetLastError();
}

// out must be zero-initialised (or hold a running sum) by the caller
int b200_colsum(const void* x, float* out, long long rows, int cols, long long ld, int is_bf16, cudaStream_t st) {
  if (rows <= 0 || cols <= 0) return 0;
  if (is_bf16 && cols % 8 == 0 && ld % 8 == 0 && ((uintptr_t)x & 15) == 0) {
    const int cb = (cols + 255) / 256;
    long long rpb = (rows * cb + 148LL * 8 - 1) / (148LL * 8);      // about 8 blocks per SM
    rpb = rpb < 32 ? 32 : rpb > 1024 ? 1024 : (rpb + 31) / 32 * 32;
    dim3 g(cb, (unsigned)((rows + rpb - 1) / rpb));
    launch_pdl(colsum_vec_kernel, g, dim3(256), 0, st, (const __nv_bfloat16*)x, out, rows, cols, ld, (int)rpb);
    return (int)cudaGetLastError();
  }
  int rpb = 256;
  dim3 grid((cols + 127) / 128, (unsigned)((rows + rpb - 1) / rpb));
  if (is_bf16) colsum_kernel<__nv_bfloat16><<<grid, 128, 0, st>>>((const __nv_bfloat16*)x, out, rows, cols, ld, rpb);
  else colsum_kernel<float><<<grid, 128, 0, st>>>((const float*)x, out, rows, cols, ld, rpb);
  return (int)cudaGetLastError();
}

// rows_valid (optional, device int [batch]): only the first rows_valid[z] rows, rounded up to 128, of batch z are summed
int b200_colsum_batched(const void* x, float* out, int batch, long long rows, int cols, long long ld, long long bs,
                        int is_bf16, const int* rows_valid, cudaStream_t st) {
  if (rows <= 0 || cols <= 0 || batch <= 0) return 0;
  dim3 grid((cols + 127) / 128, (unsigned)((rows + 255) / 256), batch);
  if (is_bf16) colsum_batched_kernel<__nv_bfloat16><<<grid, 128, 0, st>>>((const __nv_bfloat16*)x, out, rows, cols, ld, bs, rows_valid);
  else colsum_batched_kernel<float><<<grid, 128, 0, st>>>((const float*)x, out, rows, cols, ld, bs, rows_valid);
  return (int)cudaGetLastError();
}

// what: 0 sum, 1 sum of squares, 2 max, 3 min. `out` must be pre-initialised (0, 0, -inf, +inf).
int b200_reduce(const void* x, float* out, long long n, int what, int is_bf16, cudaStream_t st) {
  if (n <= 0) return 0;
  if (is_bf16) reduce_kernel<__nv_bfloat16><<<grid_for(n, 256, 592), 256, 0, st>>>((const __nv_bfloat16*)x, out, n, what);
  else reduce_kernel<float><<<grid_for(n, 256, 592), 256, 0, st>>>((const float*)x, out, n, what);
  return (int)cudaGetLastError();
}

int b200_softmax_fwd(const void* x, void* y, long long rows, int cols, float scale, int causal_period, int is_bf16, cudaStream_t st) {
  if (rows <= 0 || cols <= 0) return 0;
  const int threads = cols >= 1024 ? 256 : 128;
  if (is_bf16) softmax_fwd_kernel<__nv_bfloat16><<<(unsigned)rows, threads, 0, st>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y, cols, scale, causal_period);
  else softmax_fwd_kernel<float><<<(unsigned)rows, threads, 0, st>>>((const float*)x, (float*)y, cols, scale, causal_period);
  return (int)cudaGetLastError();
}

int b200_softmax_bwd(const void* dy, const void* y, void* dx, long long rows, int cols, float scale, int is_bf16, cudaStream_t st) {
  if (rows <= 0 || cols <= 0) return 0;
  const int threads = cols >= 1024 ? 256 : 128;
  if (is_bf16) softmax_bwd_kernel<__nv_bfloat16><<<(unsigned)rows, threads, 0, st>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)y, (__nv_bfloat16*)dx, cols, scale);
  else softmax_bwd_kernel<float><<<(unsigned)rows, threads, 0, st>>>((const float*)dy, (const float*)y, (float*)dx, cols, scale);
  return (int)cudaGetLastError();
}

// Programmatic dependent launch on (1, default) or off (0) for every kernel of this library that supports it.
int b200_set_pdl(int on) { b200::g_pdl_enabled = on ? 1 : 0; return 0; }

int b200_dropout(const void* x, void* y, long long n, float p, unsigned long long seed, int is_bf16, cudaStream_t st) {
  if (n <= 0) return 0;
  float scale = p < 1.f ? 1.f / (1.f - p) : 0.f;
  if (is_bf16) dropout_kernel<__nv_bfloat16><<<grid_for(n, 256), 256, 0, st>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y, n, p, scale, seed);
  else dropout_kernel<float><<<grid_for(n, 256), 256, 0, st>>>((const float*)x, (float*)y, n, p, scale, seed);
  return (int)cudaGetLastError();
}

int b200_fake_quant(const void* x, void* y, long long n, float scale, float qmin, float qmax, int is_bf16,
                    cudaStream_t st) {
  if (n <= 0) return 0;
  if (is_bf16) fake_quant_kernel<__nv_bfloat16><<<grid_for(n, 256), 256, 0, st>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y, n, scale, qmin, qmax);
  else fake_quant_kernel<float><<<grid_for(n, 256), 256, 0, st>>>((const float*)x, (float*)y, n, scale, qmin, qmax);
  return (int)cudaGetLastError();
}

int b200_transpose(const void* in, void* out, int rows, int cols, long long ld_in, long long ld_out, long long bs_in,
                   long long bs_out, int batch, int is_bf16, cudaStream_t st) {
  if (rows <= 0 || cols <= 0 || batch <= 0) return 0;
  dim3 grid((cols + 31) / 32, (rows + 31) / 32, batch), block(32, 8);
  if (is_bf16) transpose_kernel<__nv_bfloat16><<<grid, block, 0, st>>>((const __nv_bfloat16*)in, (__nv_bfloat16*)out, rows, cols, ld_in, ld_out, bs_in, bs_out);
  else transpose_kernel<float><<<grid, block, 0, st>>>((const float*)in, (float*)out, rows, cols, ld_in, ld_out, bs_in, bs_out);
  return (int)cudaGetLastError();
}

int b200_rope(const void* x, const float* cos_t, const float* sin_t, void* y, long long leading, int seq, int dim,
              float sign, int is_bf16, cudaStream_t st) {
  if (leading <= 0 || seq <= 0 || dim <= 0) return 0;
  long long total = leading * seq * (dim / 2);
  if (is_bf16) rope_kernel<__nv_bfloat16><<<grid_for(total, 256), 256, 0, st>>>((const __nv_bfloat16*)x, cos_t, sin_t, (__nv_bfloat16*)y, leading, seq, dim, sign);
  else rope_kernel<float><<<grid_for(total, 256), 256, 0, st>>>((const float*)x, cos_t, sin_t, (float*)y, leading, seq, dim, sign);
  return (int)cudaGetLastError();
}

int b200_embedding_fwd(const void* table, const long long* ids, void* out, long long tokens, int dim, long long vocab,
                       int is_bf16, cudaStream_t st) {
  if (tokens <= 0) return 0;
  if (is_bf16) {
    if (dim % 8) return -1;
    embedding_fwd_kernel<__nv_bfloat16><<<grid_for(tokens * (dim / 8), 256), 256, 0, st>>>((const __nv_bfloat16*)table, ids, (__nv_bfloat16*)out, tokens, dim, vocab);
  } else {
    if (dim % 4) return -1;
    embedding_fwd_kernel<float><<<grid_for(tokens * (dim / 4), 256), 256, 0, st>>>((const float*)table, ids, (float*)out, tokens, dim, vocab);
  }
  return (int)cudaGetLastError();
}

int b200_embedding_bwd(const void* g, const long long* ids, float* grad_table, long long tokens, int dim,
                       long long vocab, int is_bf16, cudaStream_t st) {
  if (tokens <= 0) return 0;
  if (is_bf16) embedding_bwd_kernel<__nv_bfloat16><<<grid_for(tokens * dim, 256), 256, 0, st>>>((const __nv_bfloat16*)g, ids, grad_table, tokens, dim, vocab);
  else embedding_bwd_kernel<float><<<grid_for(tokens * dim, 256), 256, 0, st>>>((const float*)g, ids, grad_table, tokens, dim, vocab);
  return (int)cudaGetLastError();
}

}  // extern "C"
