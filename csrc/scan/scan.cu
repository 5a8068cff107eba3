// S1/S2: Mamba (S6) selective scan forward / backward, S3: depthwise causal conv1d (+SiLU) forward / backward.
//
// Recurrence (rust-nn src/tensor.rs:833-896, backward 1710-1819):
//   h_t[d,n] = exp(delta_t[d] * A[d,n]) * h_{t-1}[d,n] + delta_t[d] * B_t[n] * u_t[d]
//   y_t[d]   = sum_n C_t[n] * h_t[d,n]   (+ Dskip[d] * u_t[d])   (* silu(z_t[d]) when a gate is given)
// with delta = softplus(delta_raw + delta_bias) when `delta_softplus` is set.
//
// A is diagonal per (channel, state), so this is not a tensor-core contraction: the kernels keep the
// fp32 state in registers, one thread per (batch, channel) with all N <= 16 states, stream u/delta/z
// through coalesced loads and B_t/C_t through shared memory, and use exp2 with log2(e) folded into A.
// The forward stores the state every CK steps; the backward walks those checkpoints in reverse,
// recomputes the CK intermediate states into shared memory and runs the adjoint recurrence -
// it never stores seq x d x n states as the reference's backward does (src/tensor.rs:1750-1802).
// dB_t / dC_t are reduced across the 32 channels of a warp with a transpose-reduce (31 shuffles for
// 32 values) and then added atomically.
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cstdint>

namespace b200 {

constexpr int SCAN_N = 16;       // max states per channel
constexpr int SCAN_CK = 8;       // checkpoint interval (steps)
constexpr int SCAN_THREADS = 128;

template <typename T> __device__ __forceinline__ float s_ld(const T* p);
template <> __device__ __forceinline__ float s_ld<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float s_ld<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void s_st(T* p, float v);
template <> __device__ __forceinline__ void s_st<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void s_st<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16(v); }

__device__ __forceinline__ float softplus20(float v) { return v > 20.f ? v : log1pf(__expf(v)); }
__device__ __forceinline__ float sigmoidf_(float v) { return 1.f / (1.f + __expf(-v)); }

struct ScanArgs {
  const void* u; long long u_ld;            // [B, S, D] rows of stride u_ld
  const void* delta; long long delta_ld;    // [B, S, D]
  const void* z; long long z_ld;            // optional gate [B, S, D]
  const void* Bm; long long b_ld;           // [B, S, N]
  const void* Cm; long long c_ld;           // [B, S, N]
  const float* A;                           // [D, N] (negative)
  const float* Dskip;                       // optional [D]
  const float* delta_bias;                  // optional [D]
  void* y; long long y_ld;                  // [B, S, D]
  float* hck;                               // checkpoints [B, ceil(S/CK), D, N] (state BEFORE step c*CK)
  int B, S, D, N;
  int delta_softplus;
  // backward
  const void* dy; long long dy_ld;
  void* du; long long du_ld;
  void* ddelta; long long ddelta_ld;
  void* dz; long long dz_ld;
  float* dB; float* dC;                     // [B, S, N] fp32, zero-initialised by the caller
  float* dA; float* dDskip; float* ddelta_bias;   // fp32 accumulators [D,N], [D], [D]
};

template <typename T>
__global__ void __launch_bounds__(SCAN_THREADS)
selective_scan_fwd_kernel(ScanArgs a) {
  const int b = blockIdx.y;
  const int d = blockIdx.x * SCAN_THREADS + threadIdx.x;
  const bool active = d < a.D;
  const int N = a.N;
  __shared__ float sB[SCAN_CK][SCAN_N], sC[SCAN_CK][SCAN_N];
  float A2[SCAN_N], h[SCAN_N];
#pragma unroll
  for (int n = 0; n < SCAN_N; ++n) {
    A2[n] = (active && n < N) ? a.A[(long long)d * N + n] * 1.4426950408889634f : 0.f;
    h[n] = 0.f;
  }
  const float dsk = (active && a.Dskip) ? a.Dskip[d] : 0.f;
  const float dbias = (active && a.delta_bias) ? a.delta_bias[d] : 0.f;
  const T* up = (const T*)a.u + (long long)b * a.S * a.u_ld + d;
  const T* dp = (const T*)a.delta + (long long)b * a.S * a.delta_ld + d;
  const T* zp = a.z ? (const T*)a.z + (long long)b * a.S * a.z_ld + d : nullptr;
  T* yp = (T*)a.y + (long long)b * a.S * a.y_ld + d;
  const T* Bp = (const T*)a.Bm + (long long)b * a.S * a.b_ld;
  const T* Cp = (const T*)a.Cm + (long long)b * a.S * a.c_ld;
  const int n_ck = (a.S + SCAN_CK - 1) / SCAN_CK;
  for (int c = 0; c < n_ck; ++c) {
    const int t0 = c * SCAN_CK;
    __syncthreads();
    for (int i = threadIdx.x; i < SCAN_CK * SCAN_N; i += SCAN_THREADS) {
      const int tt = i / SCAN_N, n = i % SCAN_N;
      const bool ok = (t0 + tt < a.S) && n < N;
      sB[tt][n] = ok ? s_ld(Bp + (long long)(t0 + tt) * a.b_ld + n) : 0.f;
      sC[tt][n] = ok ? s_ld(Cp + (long long)(t0 + tt) * a.c_ld + n) : 0.f;
    }
    __syncthreads();
    if (!active) continue;
    if (a.hck) {
      float* ck = a.hck + (((long long)b * n_ck + c) * a.D + d) * N;
#pragma unroll
      for (int n = 0; n < SCAN_N; ++n) if (n < N) ck[n] = h[n];
    }
    float uu[SCAN_CK], dd[SCAN_CK], zz[SCAN_CK];
#pragma unroll
    for (int tt = 0; tt < SCAN_CK; ++tt) {
      const bool ok = t0 + tt < a.S;
      uu[tt] = ok ? s_ld(up + (long long)(t0 + tt) * a.u_ld) : 0.f;
      dd[tt] = ok ? s_ld(dp + (long long)(t0 + tt) * a.delta_ld) : 0.f;
      zz[tt] = (ok && zp) ? s_ld(zp + (long long)(t0 + tt) * a.z_ld) : 0.f;
    }
#pragma unroll
    for (int tt = 0; tt < SCAN_CK; ++tt) {
      if (t0 + tt >= a.S) break;
      float dl = dd[tt] + dbias;
      if (a.delta_softplus) dl = softplus20(dl);
      const float du = dl * uu[tt];
      float y = dsk * uu[tt];
#pragma unroll
      for (int n = 0; n < SCAN_N; ++n) {
        h[n] = exp2f(dl * A2[n]) * h[n] + du * sB[tt][n];
        y += sC[tt][n] * h[n];
      }
      if (zp) y *= zz[tt] * sigmoidf_(zz[tt]);
      s_st(yp + (long long)(t0 + tt) * a.y_ld, y);
    }
  }
}

// Sum 32 per-lane arrays of 32 values across the warp; afterwards lane i holds the total of value i.
__device__ __forceinline__ float warp_transpose_reduce32(float (&v)[32], int lane) {
#pragma unroll
  for (int step = 0; step < 5; ++step) {
    const int half = 16 >> step;           // number of values kept after this step
    const int lane_bit = 16 >> step;
    const bool upper = (lane & lane_bit) != 0;
#pragma unroll
    for (int i = 0; i < half; ++i) {
      // lanes with the bit set keep the upper half of the remaining values, the others the lower half
      const float send = upper ? v[i] : v[i + half];
      const float keep = upper ? v[i + half] : v[i];
      v[i] = keep + __shfl_xor_sync(0xffffffffu, send, lane_bit);
    }
  }
  return v[0];
}
// index of the value that ends up in `lane` after warp_transpose_reduce32
__device__ __forceinline__ int transpose_reduce_owner(int lane) { return lane; }

template <typename T>
__global__ void __launch_bounds__(SCAN_THREADS)
selective_scan_bwd_kernel(ScanArgs a) {
  extern __shared__ float smem[];
  float* sH = smem;                                         // [CK+1][N][THREADS] states h_{t0-1} .. h_{t0+CK-1}
  float* sB = sH + (SCAN_CK + 1) * SCAN_N * SCAN_THREADS;   // [CK][N]
  float* sC = sB + SCAN_CK * SCAN_N;                        // [CK][N]
  const int b = blockIdx.y;
  const int d = blockIdx.x * SCAN_THREADS + threadIdx.x;
  const int lane = threadIdx.x & 31;
  const bool active = d < a.D;
  const int N = a.N;
  float A2[SCAN_N], Araw[SCAN_N], dh[SCAN_N], dAacc[SCAN_N];
#pragma unroll
  for (int n = 0; n < SCAN_N; ++n) {
    Araw[n] = (active && n < N) ? a.A[(long long)d * N + n] : 0.f;
    A2[n] = Araw[n] * 1.4426950408889634f;
    dh[n] = 0.f; dAacc[n] = 0.f;
  }
  const float dsk = (active && a.Dskip) ? a.Dskip[d] : 0.f;
  const float dbias = (active && a.delta_bias) ? a.delta_bias[d] : 0.f;
  float dDacc = 0.f, ddbias_acc = 0.f;
  const long long rb = (long long)b * a.S;
  const T* up = (const T*)a.u + rb * a.u_ld + d;
  const T* dp = (const T*)a.delta + rb * a.delta_ld + d;
  const T* zp = a.z ? (const T*)a.z + rb * a.z_ld + d : nullptr;
  const T* gyp = (const T*)a.dy + rb * a.dy_ld + d;
  T* dup = (T*)a.du + rb * a.du_ld + d;
  T* ddp = (T*)a.ddelta + rb * a.ddelta_ld + d;
  T* dzp = a.dz ? (T*)a.dz + rb * a.dz_ld + d : nullptr;
  const T* Bp = (const T*)a.Bm + rb * a.b_ld;
  const T* Cp = (const T*)a.Cm + rb * a.c_ld;
  const int n_ck = (a.S + SCAN_CK - 1) / SCAN_CK;
#define SH(t, n) sH[((t) * SCAN_N + (n)) * SCAN_THREADS + threadIdx.x]
  for (int c = n_ck - 1; c >= 0; --c) {
    const int t0 = c * SCAN_CK;
    __syncthreads();
    for (int i = threadIdx.x; i < SCAN_CK * SCAN_N; i += SCAN_THREADS) {
      const int tt = i / SCAN_N, n = i % SCAN_N;
      const bool ok = (t0 + tt < a.S) && n < N;
      sB[i] = ok ? s_ld(Bp + (long long)(t0 + tt) * a.b_ld + n) : 0.f;
      sC[i] = ok ? s_ld(Cp + (long long)(t0 + tt) * a.c_ld + n) : 0.f;
    }
    __syncthreads();
    float uu[SCAN_CK], dl[SCAN_CK], draw[SCAN_CK], zz[SCAN_CK], gy[SCAN_CK], yraw[SCAN_CK];
#pragma unroll
    for (int tt = 0; tt < SCAN_CK; ++tt) {
      const bool ok = active && (t0 + tt < a.S);
      uu[tt] = ok ? s_ld(up + (long long)(t0 + tt) * a.u_ld) : 0.f;
      draw[tt] = ok ? s_ld(dp + (long long)(t0 + tt) * a.delta_ld) + dbias : 0.f;
      dl[tt] = a.delta_softplus ? softplus20(draw[tt]) : draw[tt];
      if (!ok) dl[tt] = 0.f;
      zz[tt] = (ok && zp) ? s_ld(zp + (long long)(t0 + tt) * a.z_ld) : 0.f;
      gy[tt] = ok ? s_ld(gyp + (long long)(t0 + tt) * a.dy_ld) : 0.f;
    }
    // recompute the states of this chunk from its checkpoint
    if (active) {
      const float* ck = a.hck + (((long long)b * n_ck + c) * a.D + d) * N;
#pragma unroll
      for (int n = 0; n < SCAN_N; ++n) SH(0, n) = n < N ? ck[n] : 0.f;
#pragma unroll
      for (int tt = 0; tt < SCAN_CK; ++tt) {
        const float du = dl[tt] * uu[tt];
        float y = dsk * uu[tt];
#pragma unroll
        for (int n = 0; n < SCAN_N; ++n) {
          const float hn = exp2f(dl[tt] * A2[n]) * SH(tt, n) + du * sB[tt * SCAN_N + n];
          SH(tt + 1, n) = hn;
          y += sC[tt * SCAN_N + n] * hn;
        }
        yraw[tt] = y;
      }
    }
    // adjoint recurrence, reverse in time
#pragma unroll
    for (int tt = SCAN_CK - 1; tt >= 0; --tt) {
      const int t = t0 + tt;
      const bool step_ok = t < a.S;          // block-uniform
      if (!step_ok) continue;
      float g = gy[tt];
      if (zp) {
        const float sg = sigmoidf_(zz[tt]);
        const float sz = zz[tt] * sg;
        if (active && dzp) s_st(dzp + (long long)t * a.dz_ld, g * yraw[tt] * sg * (1.f + zz[tt] * (1.f - sg)));
        g *= sz;
      }
      dDacc += g * uu[tt];
      float du_t = g * dsk;
      float ddl = 0.f;
      float red[32];
#pragma unroll
      for (int n = 0; n < SCAN_N; ++n) {
        const float hprev = SH(tt, n), hcur = SH(tt + 1, n);
        const float Bn = sB[tt * SCAN_N + n], Cn = sC[tt * SCAN_N + n];
        red[SCAN_N + n] = g * hcur;                         // dC_t[n] contribution of this channel
        const float dhn = dh[n] + g * Cn;
        const float da = exp2f(dl[tt] * A2[n]);
        const float dda = dhn * hprev;
        ddl += dda * da * Araw[n] + dhn * Bn * uu[tt];
        dAacc[n] += dda * da * dl[tt];
        red[n] = dhn * dl[tt] * uu[tt];                      // dB_t[n] contribution
        du_t += dhn * dl[tt] * Bn;
        dh[n] = dhn * da;
      }
      if (!active) {
#pragma unroll
        for (int i = 0; i < 32; ++i) red[i] = 0.f;
      }
      const float total = warp_transpose_reduce32(red, lane);
      // lane i now holds the warp total of value i: i < 16 -> dB[n = i], else dC[n = i - 16]
      {
        const int n = lane & 15;
        if (n < N) {
          float* dst = (lane < 16 ? a.dB : a.dC) + (rb + t) * N + n;
          atomicAdd(dst, total);
        }
      }
      if (active) {
        float ddraw = ddl;
        if (a.delta_softplus) ddraw *= sigmoidf_(draw[tt]);
        ddbias_acc += ddraw;
        s_st(dup + (long long)t * a.du_ld, du_t);
        s_st(ddp + (long long)t * a.ddelta_ld, ddraw);
      }
    }
  }
#undef SH
  if (active) {
#pragma unroll
    for (int n = 0; n < SCAN_N; ++n) if (n < N) atomicAdd(a.dA + (long long)d * N + n, dAacc[n]);
    if (a.dDskip) atomicAdd(a.dDskip + d, dDacc);
    if (a.ddelta_bias) atomicAdd(a.ddelta_bias + d, ddbias_acc);
  }
}

// ---------------------------------------------------------------------------- lane-per-state scan (N == 16, no fused gate)
// The thread-per-channel kernels above expose B*D threads (32768 for the Mamba configuration) and every step
// waits on the previous one: they are latency-bound at a few percent of the machine. Here a lane owns ONE state
// (channel, n): a warp carries 2 channels x 16 states, 16x the threads, one MUFU ex2 and three FMAs per lane
// and step. The sum over n that y_t (forward) and d delta_t / d u_t (backward) need is taken 16 steps at a time
// with a transpose-reduce inside each half-warp (15 shuffles for 16 sums) instead of 4 shuffles per step.
// u / delta / B / C move through shared-memory tiles filled with coalesced loads while the previous tile is
// being processed. The checkpoint layout is the one of the kernels above, so either backward can follow either
// forward.
constexpr float SCAN_LOG2E = 1.4426950408889634f;
__device__ __forceinline__ float scan_ex2(float x) { float y; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }

// sums 16 per-lane values over the 16 lanes of a half-warp; lane j (mod 16) ends with the total of v[j]
__device__ __forceinline__ float transpose_reduce16(float (&v)[16], int lane) {
#pragma unroll
  for (int step = 0; step < 4; ++step) {
    const int half = 8 >> step;
    const bool upper = (lane & half) != 0;
#pragma unroll
    for (int i = 0; i < half; ++i) {
      const float send = upper ? v[i] : v[i + half];
      const float keep = upper ? v[i + half] : v[i];
      v[i] = keep + __shfl_xor_sync(0xffffffffu, send, half);
    }
  }
  return v[0];
}

template <typename T>
__global__ void __launch_bounds__(256)
scan_fwd_lanes_kernel(ScanArgs a) {
  constexpr int DB = 16, TT = 32;
  __shared__ float2 s_x[2][TT][DB];                   // (delta, delta * u)
  __shared__ float2 s_BC[2][TT][SCAN_N];
  __shared__ float s_u[2][TT][DB], s_y[TT][DB];
  const int b = blockIdx.y, d0 = blockIdx.x * DB;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = lane & 15, ch = warp * 2 + (lane >> 4);
  const int d = d0 + ch;
  const bool active = d < a.D;
  const float A2 = active ? a.A[(long long)d * SCAN_N + n] * SCAN_LOG2E : 0.f;
  const float dsk = (active && a.Dskip) ? a.Dskip[d] : 0.f;
  const int n_ck = (a.S + SCAN_CK - 1) / SCAN_CK;
  float h = 0.f;
  // loader role: thread -> (row lt of the tile, channel / state pair lp)
  const int lt = threadIdx.x >> 3, lp = threadIdx.x & 7;
  const int ld0 = d0 + 2 * lp, ld1 = ld0 + 1;
  const float db0 = (a.delta_bias && ld0 < a.D) ? a.delta_bias[ld0] : 0.f, db1 = (a.delta_bias && ld1 < a.D) ? a.delta_bias[ld1] : 0.f;
  const long long rb = (long long)b * a.S;
  const T* up = (const T*)a.u; const T* dp = (const T*)a.delta; const T* Bp = (const T*)a.Bm; const T* Cp = (const T*)a.Cm;
  float r[8];
  auto load_tile = [&](int t0) {
    const int t = t0 + lt;
    const bool ok = t < a.S;
    const long long row = rb + t;
    r[0] = (ok && ld0 < a.D) ? s_ld(up + row * a.u_ld + ld0) : 0.f;
    r[1] = (ok && ld1 < a.D) ? s_ld(up + row * a.u_ld + ld1) : 0.f;
    float x0 = (ok && ld0 < a.D) ? s_ld(dp + row * a.delta_ld + ld0) + db0 : 0.f;
    float x1 = (ok && ld1 < a.D) ? s_ld(dp + row * a.delta_ld + ld1) + db1 : 0.f;
    if (a.delta_softplus) { x0 = softplus20(x0); x1 = softplus20(x1); }
    r[2] = (ok && ld0 < a.D) ? x0 : 0.f; r[3] = (ok && ld1 < a.D) ? x1 : 0.f;
    r[4] = ok ? s_ld(Bp + row * a.b_ld + 2 * lp) : 0.f; r[5] = ok ? s_ld(Bp + row * a.b_ld + 2 * lp + 1) : 0.f;
    r[6] = ok ? s_ld(Cp + row * a.c_ld + 2 * lp) : 0.f; r[7] = ok ? s_ld(Cp + row * a.c_ld + 2 * lp + 1) : 0.f;
  };
  auto put_tile = [&](int buf) {
    s_u[buf][lt][2 * lp] = r[0]; s_u[buf][lt][2 * lp + 1] = r[1];
    s_x[buf][lt][2 * lp] = make_float2(r[2], r[2] * r[0]); s_x[buf][lt][2 * lp + 1] = make_float2(r[3], r[3] * r[1]);
    s_BC[buf][lt][2 * lp] = make_float2(r[4], r[6]); s_BC[buf][lt][2 * lp + 1] = make_float2(r[5], r[7]);
  };
  const int n_tiles = (a.S + TT - 1) / TT;
  load_tile(0); put_tile(0);
  __syncthreads();
  for (int tile = 0; tile < n_tiles; ++tile) {
    const int cur = tile & 1, t0 = tile * TT;
    if (tile + 1 < n_tiles) load_tile(t0 + TT);            // in flight while this tile is processed
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      float p[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const int t = half * 16 + i;
        if ((t % SCAN_CK) == 0 && a.hck && active && t0 + t < a.S)
          a.hck[(((long long)b * n_ck + (t0 + t) / SCAN_CK) * a.D + d) * SCAN_N + n] = h;      // state BEFORE step t
        const float2 x = s_x[cur][t][ch], bc = s_BC[cur][t][n];
        h = fmaf(scan_ex2(x.x * A2), h, x.y * bc.x);
        p[i] = h * bc.y;
      }
      const float y = transpose_reduce16(p, lane);         // lane n: sum over the states for step half*16 + n
      const int t = half * 16 + n;
      s_y[t][ch] = y + dsk * s_u[cur][t][ch];
    }
    __syncthreads();
    {
      const int t = t0 + lt;
      if (t < a.S) {
        T* yp = (T*)a.y + (rb + t) * a.y_ld;
        if (ld0 < a.D) s_st(yp + ld0, s_y[lt][2 * lp]);
        if (ld1 < a.D) s_st(yp + ld1, s_y[lt][2 * lp + 1]);
      }
    }
    if (tile + 1 < n_tiles) put_tile(cur ^ 1);
    __syncthreads();
  }
}

// Backward. A block owns 64 channels and walks the checkpoint intervals from the last to the first. Per interval
// each lane re-runs 8 steps of its state from the checkpoint, then runs the adjoint recurrence in reverse; it does so
// for 4 channels in turn (pass p: channel p*16 + 2*warp + lane/16) so that the per-(t, n) sums dB / dC, which run
// over ALL channels, gather 4 channels in registers before they touch shuffles, shared memory and finally one atomic
// per (t, n) and block. The next interval's u / delta / dy / B / C rows and checkpoints are fetched into registers
// while the current one is processed.
template <typename T>
__global__ void __launch_bounds__(256, 2)
scan_bwd_lanes_kernel(ScanArgs a) {
  constexpr int DB = 64, CK = SCAN_CK, WARPS = 8, PASSES = 4;
  __shared__ float4 s_in[CK][DB];                    // (delta, delta * u, u, dy) per (t, channel)
  __shared__ float s_draw[CK][DB];                   // delta before softplus
  __shared__ float2 s_BC[CK][SCAN_N];
  __shared__ float2 s_out[CK][DB];                   // (d delta_raw, d u without the skip term)
  __shared__ float2 s_dBC[WARPS][CK][SCAN_N];
  const int b = blockIdx.y, d0 = blockIdx.x * DB;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = lane & 15, chw = warp * 2 + (lane >> 4);     // channel inside a pass
  const int n_ck = (a.S + CK - 1) / CK;
  const long long rb = (long long)b * a.S;
  float Araw[PASSES], g_acc[PASSES], dA_acc[PASSES], ddb_acc[PASSES], dD_acc[PASSES], hnext[PASSES];
#pragma unroll
  for (int p = 0; p < PASSES; ++p) {
    const int d = d0 + p * 16 + chw;
    Araw[p] = d < a.D ? a.A[(long long)d * SCAN_N + n] : 0.f;
    g_acc[p] = dA_acc[p] = ddb_acc[p] = dD_acc[p] = 0.f;
  }
  // loader / storer role: rows lt and lt + 4 of channel lc; threads 0..127 also fetch B, 128..255 C
  const int lc = threadIdx.x & 63, lt = threadIdx.x >> 6;
  const int ldd = d0 + lc;
  const bool ch_ok = ldd < a.D;
  const float dbias = (a.delta_bias && ch_ok) ? a.delta_bias[ldd] : 0.f;
  const float dsk = (a.Dskip && ch_ok) ? a.Dskip[ldd] : 0.f;
  const int bt = (threadIdx.x & 127) >> 4, bn = threadIdx.x & 15;
  float pu[2], pd[2], pg[2], pbc;
  auto prefetch = [&](int c) {
    const int t0 = c * CK;
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int t = t0 + lt + 4 * k;
      const bool ok = t < a.S && ch_ok;
      const long long row = rb + t;
      pu[k] = ok ? s_ld((const T*)a.u + row * a.u_ld + ldd) : 0.f;
      pd[k] = ok ? s_ld((const T*)a.delta + row * a.delta_ld + ldd) : 0.f;
      pg[k] = ok ? s_ld((const T*)a.dy + row * a.dy_ld + ldd) : 0.f;
    }
    const bool okb = t0 + bt < a.S;
    if (threadIdx.x < 128) pbc = okb ? s_ld((const T*)a.Bm + (rb + t0 + bt) * a.b_ld + bn) : 0.f;
    else pbc = okb ? s_ld((const T*)a.Cm + (rb + t0 + bt) * a.c_ld + bn) : 0.f;
#pragma unroll
    for (int p = 0; p < PASSES; ++p) {
      const int d = d0 + p * 16 + chw;
      hnext[p] = d < a.D ? a.hck[(((long long)b * n_ck + c) * a.D + d) * SCAN_N + n] : 0.f;
    }
  };
  prefetch(n_ck - 1);
  for (int c = n_ck - 1; c >= 0; --c) {
    const int t0 = c * CK;
    __syncthreads();                                  // the previous interval's tiles are no longer read
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int t = t0 + lt + 4 * k;
      const bool ok = t < a.S && ch_ok;
      const float draw = ok ? pd[k] + dbias : 0.f;
      const float dl = ok ? (a.delta_softplus ? softplus20(draw) : draw) : 0.f;
      s_in[lt + 4 * k][lc] = make_float4(dl, dl * pu[k], pu[k], pg[k]);
      s_draw[lt + 4 * k][lc] = draw;
    }
    if (threadIdx.x < 128) s_BC[bt][bn].x = pbc; else s_BC[bt][bn].y = pbc;
    float h0[PASSES];
#pragma unroll
    for (int p = 0; p < PASSES; ++p) h0[p] = hnext[p];
    __syncthreads();
    if (c > 0) prefetch(c - 1);                       // in flight during the passes below
    float dBp[CK], dCp[CK];
#pragma unroll
    for (int i = 0; i < CK; ++i) dBp[i] = dCp[i] = 0.f;
#pragma unroll
    for (int p = 0; p < PASSES; ++p) {
      const int ch = p * 16 + chw;
      const float A2 = Araw[p] * SCAN_LOG2E;
      float hs[CK + 1], av[CK];
      hs[0] = h0[p];
#pragma unroll
      for (int i = 0; i < CK; ++i) {
        const float4 x = s_in[i][ch];
        av[i] = scan_ex2(x.x * A2);
        hs[i + 1] = fmaf(av[i], hs[i], x.y * s_BC[i][n].x);
      }
      float red[16];
      float g = g_acc[p], dA = dA_acc[p];
#pragma unroll
      for (int i = CK - 1; i >= 0; --i) {
        const float4 x = s_in[i][ch];                 // (dl, dl*u, u, gy)
        const float2 bc = s_BC[i][n];
        const float dhn = fmaf(x.w, bc.y, g);
        const float t1 = dhn * hs[i] * av[i];
        const float xb = dhn * bc.x;
        red[i] = fmaf(t1, Araw[p], xb * x.z);         // d delta_t, this state's share
        red[CK + i] = xb * x.x;                       // d u_t, this state's share
        dA = fmaf(t1, x.x, dA);
        dBp[i] = fmaf(dhn, x.y, dBp[i]);
        dCp[i] = fmaf(x.w, hs[i + 1], dCp[i]);
        g = dhn * av[i];
      }
      g_acc[p] = g; dA_acc[p] = dA;
      const float tot = transpose_reduce16(red, lane);   // lane j < 8: d delta of step j; j >= 8: d u of step j - 8
      const int j = lane & 15;
      if (j < CK) {
        float ddraw = tot;
        if (a.delta_softplus) ddraw *= sigmoidf_(s_draw[j][ch]);
        s_out[j][ch].x = ddraw;
        ddb_acc[p] += ddraw;
        const float4 x = s_in[j][ch];
        dD_acc[p] = fmaf(x.w, x.z, dD_acc[p]);
      } else {
        s_out[j - CK][ch].y = tot;
      }
    }
#pragma unroll
    for (int i = 0; i < CK; ++i) {
      dBp[i] += __shfl_xor_sync(0xffffffffu, dBp[i], 16);    // the warp's two channel groups
      dCp[i] += __shfl_xor_sync(0xffffffffu, dCp[i], 16);
      if (lane < 16) s_dBC[warp][i][n] = make_float2(dBp[i], dCp[i]);
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int tt = lt + 4 * k, t = t0 + tt;
      if (t < a.S && ch_ok) {
        const float2 o = s_out[tt][lc];
        s_st((T*)a.ddelta + (rb + t) * a.ddelta_ld + ldd, o.x);
        s_st((T*)a.du + (rb + t) * a.du_ld + ldd, fmaf(dsk, s_in[tt][lc].w, o.y));
      }
    }
    if (t0 + bt < a.S) {
      float acc = 0.f;
      if (threadIdx.x < 128) {
#pragma unroll
        for (int w = 0; w < WARPS; ++w) acc += s_dBC[w][bt][bn].x;
        atomicAdd(a.dB + (rb + t0 + bt) * SCAN_N + bn, acc);
      } else {
#pragma unroll
        for (int w = 0; w < WARPS; ++w) acc += s_dBC[w][bt][bn].y;
        atomicAdd(a.dC + (rb + t0 + bt) * SCAN_N + bn, acc);
      }
    }
  }
#pragma unroll
  for (int p = 0; p < PASSES; ++p) {
    const int d = d0 + p * 16 + chw;
    float v0 = ddb_acc[p], v1 = dD_acc[p];            // per-channel sums sit in lanes j < 8 of each half-warp
#pragma unroll
    for (int o = 8; o; o >>= 1) { v0 += __shfl_xor_sync(0xffffffffu, v0, o); v1 += __shfl_xor_sync(0xffffffffu, v1, o); }
    if (d < a.D) {
      atomicAdd(a.dA + (long long)d * SCAN_N + n, dA_acc[p]);
      if (n == 0) {
        if (a.ddelta_bias) atomicAdd(a.ddelta_bias + d, v0);
        if (a.dDskip) atomicAdd(a.dDskip + d, v1);
      }
    }
  }
}

// ---------------------------------------------------------------------------- causal depthwise conv1d
// y[b,t,c] = act( bias[c] + sum_k w[c,k] * x[b, t-(K-1)+k, c] ), K <= 8, act in {none, silu}
// (rust-nn src/tensor.rs:903-944; its MambaBlock applies SiLU right after, src/mamba.rs:95-98)
constexpr int CONV_MAXK = 8;
constexpr int CONV_TCHUNK = 64;

template <typename T, int K>
__global__ void conv1d_fwd_kernel(const T* __restrict__ x, long long x_ld, const float* __restrict__ w,
                                  const float* __restrict__ bias, T* __restrict__ y, long long y_ld, int B, int S, int C,
                                  int act) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int b = blockIdx.z;
  const int t0 = blockIdx.y * CONV_TCHUNK;
  if (c >= C) return;
  float wk[K], win[K];
#pragma unroll
  for (int k = 0; k < K; ++k) wk[k] = w[c * K + k];
  const float bs = bias ? bias[c] : 0.f;
  const T* xp = x + (long long)b * S * x_ld + c;
  T* yp = y + (long long)b * S * y_ld + c;
  // win[k] holds x[t-(K-1)+k]
#pragma unroll
  for (int k = 0; k < K - 1; ++k) {
    const int t = t0 - (K - 1) + k;
    win[k] = t >= 0 ? s_ld(xp + (long long)t * x_ld) : 0.f;
  }
  const int t1 = min(t0 + CONV_TCHUNK, S);
  for (int t = t0; t < t1; ++t) {
    win[K - 1] = s_ld(xp + (long long)t * x_ld);
    float acc = bs;
#pragma unroll
    for (int k = 0; k < K; ++k) acc += wk[k] * win[k];
    if (act) acc = acc * sigmoidf_(acc);
    s_st(yp + (long long)t * y_ld, acc);
#pragma unroll
    for (int k = 0; k < K - 1; ++k) win[k] = win[k + 1];
  }
}

// dx[b,t,c] = sum_k w[c,k] * dpre[b, t+(K-1)-k, c];  dw[c,k] += sum dpre[t] x[t-(K-1)+k];  dbias[c] += sum dpre[t]
// with dpre = dy * act'(pre), pre recomputed from x.
template <typename T, int K>
__global__ void conv1d_bwd_kernel(const T* __restrict__ x, long long x_ld, const float* __restrict__ w,
                                  const float* __restrict__ bias, const T* __restrict__ dy, long long dy_ld,
                                  T* __restrict__ dx, long long dx_ld, float* __restrict__ dw, float* __restrict__ dbias,
                                  int B, int S, int C, int act) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int b = blockIdx.z;
  const int t0 = blockIdx.y * CONV_TCHUNK;
  if (c >= C) return;
  float wk[K], dwk[K];
#pragma unroll
  for (int k = 0; k < K; ++k) { wk[k] = w[c * K + k]; dwk[k] = 0.f; }
  const float bs = bias ? bias[c] : 0.f;
  const T* xp = x + (long long)b * S * x_ld + c;
  const T* gp = dy + (long long)b * S * dy_ld + c;
  T* dxp = dx + (long long)b * S * dx_ld + c;
  const int t1 = min(t0 + CONV_TCHUNK, S);
  float dbacc = 0.f;
  // Sliding windows, one new x and one new dy per time step:
  //   xw[i]   = x[t - (K-1) + i], i in [0, 2K-1)   (0 outside [0, S)): covers the taps of dpre[t + K-1] and of dw at t
  //   dwin[i] = dpre[t + i],      i in [0, K)        with dpre = dy * act'(pre), pre recomputed from the window
  float xw[2 * K - 1], dwin[K];
#pragma unroll
  for (int i = 0; i < 2 * K - 2; ++i) { const int tx = t0 - (K - 1) + i; xw[i] = (tx >= 0 && tx < S) ? s_ld(xp + (long long)tx * x_ld) : 0.f; }
  auto dpre_from = [&](int t, const float* xtaps) -> float {          // xtaps[j] = x[t - (K-1) + j]
    if (t >= S) return 0.f;
    const float g = s_ld(gp + (long long)t * dy_ld);
    if (!act) return g;
    float pre = bs;
#pragma unroll
    for (int j = 0; j < K; ++j) pre = fmaf(wk[j], xtaps[j], pre);
    const float sg = sigmoidf_(pre);
    return g * sg * (1.f + pre * (1.f - sg));
  };
#pragma unroll
  for (int k = 0; k < K - 1; ++k) dwin[k] = dpre_from(t0 + k, xw + k);
  for (int t = t0; t < t1; ++t) {
    const int tn = t + K - 1;
    xw[2 * K - 2] = tn < S ? s_ld(xp + (long long)tn * x_ld) : 0.f;
    dwin[K - 1] = dpre_from(tn, xw + K - 1);
    float acc = 0.f;
#pragma unroll
    for (int k = 0; k < K; ++k) acc = fmaf(wk[k], dwin[K - 1 - k], acc);
    s_st(dxp + (long long)t * dx_ld, acc);
    const float dp = dwin[0];                              // dpre[t] against x[t - (K-1) + k] = xw[k]
    dbacc += dp;
#pragma unroll
    for (int k = 0; k < K; ++k) dwk[k] = fmaf(dp, xw[k], dwk[k]);
#pragma unroll
    for (int k = 0; k < K - 1; ++k) dwin[k] = dwin[k + 1];
#pragma unroll
    for (int i = 0; i < 2 * K - 2; ++i) xw[i] = xw[i + 1];
  }
#pragma unroll
  for (int k = 0; k < K; ++k) atomicAdd(dw + c * K + k, dwk[k]);
  if (dbias) atomicAdd(dbias + c, dbacc);
}

template <typename T, int K>
static void conv_fwd_launch(const void* x, long long x_ld, const float* w, const float* bias, void* y, long long y_ld,
                            int B, int S, int C, int act, cudaStream_t st) {
  dim3 grid((C + 127) / 128, (S + CONV_TCHUNK - 1) / CONV_TCHUNK, B);
  conv1d_fwd_kernel<T, K><<<grid, 128, 0, st>>>((const T*)x, x_ld, w, bias, (T*)y, y_ld, B, S, C, act);
}
template <typename T, int K>
static void conv_bwd_launch(const void* x, long long x_ld, const float* w, const float* bias, const void* dy,
                            long long dy_ld, void* dx, long long dx_ld, float* dw, float* dbias, int B, int S, int C,
                            int act, cudaStream_t st) {
  dim3 grid((C + 127) / 128, (S + CONV_TCHUNK - 1) / CONV_TCHUNK, B);
  conv1d_bwd_kernel<T, K><<<grid, 128, 0, st>>>((const T*)x, x_ld, w, bias, (const T*)dy, dy_ld, (T*)dx, dx_ld, dw, dbias, B, S, C, act);
}

}  // namespace b200

using namespace b200;

extern "C" {

int b200_scan_ck() { return SCAN_CK; }

int b200_selective_scan_fwd(const ScanArgs* a, int is_bf16, cudaStream_t st) {
  if (a->B <= 0 || a->S <= 0 || a->D <= 0) return 0;
  if (a->N < 1 || a->N > SCAN_N) return -1;
  dim3 grid((a->D + SCAN_THREADS - 1) / SCAN_THREADS, a->B);
  if (a->N == SCAN_N && !a->z) {       // lane-per-state kernel
    dim3 g2((a->D + 15) / 16, a->B);
    if (is_bf16) scan_fwd_lanes_kernel<__nv_bfloat16><<<g2, 256, 0, st>>>(*a);
    else scan_fwd_lanes_kernel<float><<<g2, 256, 0, st>>>(*a);
    return (int)cudaGetLastError();
  }
  if (is_bf16) selective_scan_fwd_kernel<__nv_bfloat16><<<grid, SCAN_THREADS, 0, st>>>(*a);
  else selective_scan_fwd_kernel<float><<<grid, SCAN_THREADS, 0, st>>>(*a);
  return (int)cudaGetLastError();
}

int b200_selective_scan_bwd(const ScanArgs* a, int is_bf16, cudaStream_t st) {
  if (a->B <= 0 || a->S <= 0 || a->D <= 0) return 0;
  if (a->N < 1 || a->N > SCAN_N || !a->hck) return -1;
  if (a->N == SCAN_N && !a->z) {       // lane-per-state kernel
    dim3 g2((a->D + 63) / 64, a->B);
    if (is_bf16) scan_bwd_lanes_kernel<__nv_bfloat16><<<g2, 256, 0, st>>>(*a);
    else scan_bwd_lanes_kernel<float><<<g2, 256, 0, st>>>(*a);
    return (int)cudaGetLastError();
  }
  dim3 grid((a->D + SCAN_THREADS - 1) / SCAN_THREADS, a->B);
  const int smem = ((SCAN_CK + 1) * SCAN_N * SCAN_THREADS + 2 * SCAN_CK * SCAN_N) * sizeof(float);
  static bool attr = false;
  if (!attr) {
    (void)cudaGetLastError();
    if (cudaFuncSetAttribute(selective_scan_bwd_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return -2;
    if (cudaFuncSetAttribute(selective_scan_bwd_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return -2;
    attr = true;
  }
  if (is_bf16) selective_scan_bwd_kernel<__nv_bfloat16><<<grid, SCAN_THREADS, smem, st>>>(*a);
  else selective_scan_bwd_kernel<float><<<grid, SCAN_THREADS, smem, st>>>(*a);
  return (int)cudaGetLastError();
}

#define B200_CONV_SWITCH(FN, T, ...) \
  switch (K) { case 1: FN<T, 1>(__VA_ARGS__); break; case 2: FN<T, 2>(__VA_ARGS__); break; case 3: FN<T, 3>(__VA_ARGS__); break; \
    case 4: FN<T, 4>(__VA_ARGS__); break; case 5: FN<T, 5>(__VA_ARGS__); break; case 6: FN<T, 6>(__VA_ARGS__); break; \
    case 7: FN<T, 7>(__VA_ARGS__); break; default: FN<T, 8>(__VA_ARGS__); break; }

int b200_conv1d_fwd(const void* x, long long x_ld, const float* w, const float* bias, void* y, long long y_ld, int B,
                    int S, int C, int K, int act, int is_bf16, cudaStream_t st) {
  if (B <= 0 || S <= 0 || C <= 0) return 0;
  if (K < 1 || K > CONV_MAXK) return -1;
  if (is_bf16) { B200_CONV_SWITCH(conv_fwd_launch, __nv_bfloat16, x, x_ld, w, bias, y, y_ld, B, S, C, act, st) }
  else { B200_CONV_SWITCH(conv_fwd_launch, float, x, x_ld, w, bias, y, y_ld, B, S, C, act, st) }
  return (int)cudaGetLastError();
}

int b200_conv1d_bwd(const void* x, long long x_ld, const float* w, const float* bias, const void* dy, long long dy_ld,
                    void* dx, long long dx_ld, float* dw, float* dbias, int B, int S, int C, int K, int act, int is_bf16,
                    cudaStream_t st) {
  if (B <= 0 || S <= 0 || C <= 0) return 0;
  if (K < 1 || K > CONV_MAXK) return -1;
  if (is_bf16) { B200_CONV_SWITCH(conv_bwd_launch, __nv_bfloat16, x, x_ld, w, bias, dy, dy_ld, dx, dx_ld, dw, dbias, B, S, C, act, st) }
  else { B200_CONV_SWITCH(conv_bwd_launch, float, x, x_ld, w, bias, dy, dy_ld, dx, dx_ld, dw, dbias, B, S, C, act, st) }
  return (int)cudaGetLastError();
}

}  // extern "C"
