// Block-scaled GEMM on the 5th-generation tensor cores: C[M,N] = alpha * (A .* SFA) (B .* SFB)^T with one scale factor per
// short run of K, applied by the MMA itself (`tcgen05.mma ... .block_scale`, scale factors in tensor memory).
//
//   kind 0  MXFP8 : e4m3 elements, one ue8m0 (power-of-two) scale per 32 elements   (kind::mxf8f6f4, K = 32 per MMA)
//   kind 1  NVFP4 : e2m1 elements, two per byte (low nibble first, the nibble order and magnitude table of rust-nn
//                   src/quantize.rs:139-165), one ue4m3 scale per 16 elements        (kind::mxf4nvf4, K = 64 per MMA)
//
// The reference keeps one fp32 scale per group and dequantises in software (src/quantize.rs:97-215); here the 8- and
// 4-bit operands go to the tensor core as they are and the accumulator is fp32.
//
// Operand layout. A is [M, K] and B is [N, K], both K-major, rows of K (kind 0) or K/2 (kind 1) bytes. Scale factors live
// in 512-byte chunks: a chunk holds the 4 consecutive scale factors (along K) of 128 consecutive rows, byte
// (r % 32) * 16 + (r / 32) * 4 + j for row r and scale j. Chunks are ordered [row block of 128][chunk along K]. That is
// the order `tcgen05.cp.32x128b.warpx4` wants: one copy moves a chunk into 4 TMEM columns (lane r % 32, column r / 32,
// byte j), replicated over the four lane quadrants, where the MMA reads it.
//
// Kernel: persistent, one 128 x 256 tile at a time per CTA. Warp 0 is the producer (TMA tiles of A and B with the
// 128-byte swizzle, plain bulk copies of the scale chunks, all on one mbarrier per stage), warp 1 issues the scale copies
// and the MMAs, warps 2-5 drain the accumulator (256 TMEM columns) to global memory. Every wait is bounded and reports
// through the status word.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <cstdint>

#include "../common/ptx.cuh"
#include "../common/tensormap.h"

namespace b200 {

struct MxGemmArgs {
  const void* A; const void* B;        // element bytes, K-major
  const void* sfa; const void* sfb;    // scale chunks (see above); row blocks padded to a multiple of 256 rows
  void* C; long long ldc;              // [M, N] bf16 or fp32
  int M, N, K;
  int out_f32;
  float alpha;                         // product of the per-tensor scales (NVFP4) or 1
  int kind;
  uint32_t* status;
};

template <int KIND>
struct MxCfg {
  static constexpr int BM = 128, BN = 256, BKB = 128;                 // BKB: bytes of K per row and stage
  static constexpr int K_PER_STAGE = KIND == 0 ? 128 : 256;           // elements
  static constexpr int SF_CH = KIND == 0 ? 1 : 4;                     // chunks per 128 rows and stage
  static constexpr int A_BYTES = BM * BKB, B_BYTES = BN * BKB;
  static constexpr int SFA_BYTES = 512 * SF_CH, SFB_BYTES = 2 * 512 * SF_CH;
  static constexpr int STAGE_BYTES = (A_BYTES + B_BYTES + SFA_BYTES + SFB_BYTES + 1023) / 1024 * 1024;
  static constexpr int TX_BYTES = A_BYTES + B_BYTES + SFA_BYTES + SFB_BYTES;
  static constexpr int STAGES = 4;
  static constexpr int SF_COLS = KIND == 0 ? 16 : 48;                 // TMEM columns of scale factors per stage (A: 4 * SF_CH, B: 8 * SF_CH)
  static constexpr int SMEM = STAGES * STAGE_BYTES + 256 + 1024;
};

constexpr int MX_THREADS = 192;

// shared-memory descriptor of one scale chunk: 32 rows of 16 bytes, no swizzle, 8-row groups 128 bytes apart
__device__ __forceinline__ uint64_t mx_sf_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr >> 4) & 0x3FFF);
  d |= static_cast<uint64_t>(1) << 16;          // leading-dimension offset (one 16-byte column only): 16 B
  d |= static_cast<uint64_t>(128 >> 4) << 32;   // stride between 8-row groups
  d |= static_cast<uint64_t>(1) << 46;          // descriptor version for sm_100
  return d;
}
__device__ __forceinline__ void mx_sf_copy(uint32_t taddr, uint64_t desc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(desc) : "memory");
}
__device__ __forceinline__ void bulk_load(void* smem, const void* gmem, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(smem)), "l"(reinterpret_cast<uint64_t>(gmem)), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
template <int KIND>
__device__ __forceinline__ void umma_block_scaled(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t sfa,
                                                  uint32_t sfb, uint32_t accumulate) {
  if (KIND == 0) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb) : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], p;\n\t}\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb) : "memory");
  }
}
// instruction descriptor of the block-scaled kinds: element formats at bits 7 and 10, N >> 3 at 17, scale format (1: ue8m0)
// at 23, M >> 4 at 24, the byte of the scale column each operand uses at bits 4 (B) and 29 (A); both operands K-major
template <int KIND>
__host__ __device__ constexpr uint32_t mx_idesc(uint32_t M, uint32_t N, uint32_t sf_id) {
  return (sf_id << 4) | ((KIND == 0 ? 0u : 1u) << 7) | ((KIND == 0 ? 0u : 1u) << 10) | ((N >> 3) << 17) |
         ((KIND == 0 ? 1u : 0u) << 23) | ((M >> 4) << 24) | (sf_id << 29);
}

template <int KIND>
__global__ void __launch_bounds__(MX_THREADS, 1)
gemm_mx_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const MxGemmArgs p) {
  using Cf = MxCfg<KIND>;
  constexpr int STAGES = Cf::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * Cf::STAGE_BYTES);
  uint64_t* full_bar = bars;                    // [STAGES]
  uint64_t* empty_bar = bars + STAGES;          // [STAGES]
  uint64_t* acc_full = bars + 2 * STAGES;
  uint64_t* acc_empty = bars + 2 * STAGES + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 2);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  const int m_blocks = (p.M + Cf::BM - 1) / Cf::BM, n_blocks = (p.N + Cf::BN - 1) / Cf::BN;
  const int num_kb = p.K / Cf::K_PER_STAGE;
  const int sf_chunks_k = num_kb * Cf::SF_CH;                      // chunks along K per row block
  const long long total_tiles = (long long)m_blocks * n_blocks;

  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; ++i) { mbar_init(&full_bar[i], 1); mbar_init(&empty_bar[i], 1); }
    mbar_init(acc_full, 1); mbar_init(acc_empty, 4);
    fence_barrier_init();
    tma_prefetch_desc(&tmA); tma_prefetch_desc(&tmB);
  }
  if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0; bool ok = true;
      for (long long t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        const int mb = (int)(t / n_blocks), nb = (int)(t % n_blocks);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, p.status, ST_TIMEOUT_TMA_EMPTY)) { ok = false; break; }
          uint8_t* sa = smem + stage * Cf::STAGE_BYTES;
          uint8_t* sb = sa + Cf::A_BYTES;
          uint8_t* ssfa = sb + Cf::B_BYTES;
          uint8_t* ssfb = ssfa + Cf::SFA_BYTES;
          mbar_expect_tx(&full_bar[stage], Cf::TX_BYTES);
          tma_load_3d(sa, &tmA, &full_bar[stage], kb * Cf::BKB, mb * Cf::BM, 0);
          tma_load_3d(sb, &tmB, &full_bar[stage], kb * Cf::BKB, nb * Cf::BN, 0);
          const uint8_t* ga = reinterpret_cast<const uint8_t*>(p.sfa) + ((long long)mb * sf_chunks_k + (long long)kb * Cf::SF_CH) * 512;
          bulk_load(ssfa, ga, Cf::SFA_BYTES, &full_bar[stage]);
#pragma unroll
          for (int hb = 0; hb < 2; ++hb) {
            const uint8_t* gb = reinterpret_cast<const uint8_t*>(p.sfb) + ((long long)(2 * nb + hb) * sf_chunks_k + (long long)kb * Cf::SF_CH) * 512;
            bulk_load(ssfb + hb * (Cf::SFB_BYTES / 2), gb, Cf::SFB_BYTES / 2, &full_bar[stage]);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ scale copies + MMA issue
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0, acc_phase = 0; bool ok = true;
      for (long long t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        if (!mbar_wait(acc_empty, acc_phase ^ 1, p.status, ST_TIMEOUT_ACC_EMPTY)) { ok = false; break; }
        tc_fence_after_sync();
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, p.status, ST_TIMEOUT_TMA_FULL)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem + stage * Cf::STAGE_BYTES);
          const uint32_t sb = sa + Cf::A_BYTES, ssfa = sb + Cf::B_BYTES, ssfb = ssfa + Cf::SFA_BYTES;
          const uint32_t t_sfa = tmem_base + 256 + stage * Cf::SF_COLS, t_sfb = t_sfa + 4 * Cf::SF_CH;
#pragma unroll
          for (int ch = 0; ch < Cf::SF_CH; ++ch) {
            mx_sf_copy(t_sfa + 4 * ch, mx_sf_desc(ssfa + 512 * ch));
#pragma unroll
            for (int hb = 0; hb < 2; ++hb) mx_sf_copy(t_sfb + 8 * ch + 4 * hb, mx_sf_desc(ssfb + hb * (Cf::SFB_BYTES / 2) + 512 * ch));
          }
          const uint32_t a_lo = sdesc_lo(sa, 0), b_lo = sdesc_lo(sb, 0);
#pragma unroll
          for (int j = 0; j < 4; ++j) {                       // 32 bytes of K per MMA in both kinds
            const uint32_t idesc = mx_idesc<KIND>(Cf::BM, Cf::BN, KIND == 0 ? (uint32_t)j : 0u);
            const uint32_t sfa = KIND == 0 ? t_sfa : t_sfa + 4 * j, sfb = KIND == 0 ? t_sfb : t_sfb + 8 * j;
            umma_block_scaled<KIND>(tmem_base, sdesc_at<1024>(a_lo, j * 32), sdesc_at<1024>(b_lo, j * 32), idesc, sfa, sfb,
                                    (kb > 0 || j > 0) ? 1u : 0u);
          }
          tc_commit(&empty_bar[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) tc_commit(acc_full);
        acc_phase ^= 1;
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue: warp w drains TMEM lanes 32 * (w % 4) ..
    const int quad = warp & 3;
    uint32_t acc_phase = 0; bool ok = true;
    for (long long t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
      const int mb = (int)(t / n_blocks), nb = (int)(t % n_blocks);
      if (!mbar_wait(acc_full, acc_phase, p.status, ST_TIMEOUT_ACC_FULL)) { ok = false; break; }
      tc_fence_after_sync();
      const int row = mb * Cf::BM + quad * 32 + lane;
      const uint32_t trow = tmem_base + (uint32_t(quad * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < Cf::BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_x32(trow + c * 32, r);
        tmem_ld_wait();
        const int col0 = nb * Cf::BN + c * 32;
        if (row < p.M && col0 < p.N) {
          if (p.out_f32) {
            float* cp = reinterpret_cast<float*>(p.C) + (long long)row * p.ldc + col0;
#pragma unroll
            for (int i = 0; i < 32; i += 4)
              if (col0 + i < p.N)
                *reinterpret_cast<float4*>(cp + i) = make_float4(__uint_as_float(r[i]) * p.alpha, __uint_as_float(r[i + 1]) * p.alpha,
                                                                 __uint_as_float(r[i + 2]) * p.alpha, __uint_as_float(r[i + 3]) * p.alpha);
          } else {
            __nv_bfloat16* cp = reinterpret_cast<__nv_bfloat16*>(p.C) + (long long)row * p.ldc + col0;
#pragma unroll
            for (int i = 0; i < 32; i += 8)
              if (col0 + i < p.N)
                *reinterpret_cast<uint4*>(cp + i) =
                    make_uint4(pack_bf16x2(__uint_as_float(r[i]) * p.alpha, __uint_as_float(r[i + 1]) * p.alpha),
                               pack_bf16x2(__uint_as_float(r[i + 2]) * p.alpha, __uint_as_float(r[i + 3]) * p.alpha),
                               pack_bf16x2(__uint_as_float(r[i + 4]) * p.alpha, __uint_as_float(r[i + 5]) * p.alpha),
                               pack_bf16x2(__uint_as_float(r[i + 6]) * p.alpha, __uint_as_float(r[i + 7]) * p.alpha));
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty);
      acc_phase ^= 1;
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) { tc_fence_after_sync(); tmem_dealloc(tmem_base, 512); }
}

// ---------------------------------------------------------------------------------------------------- quantise / dequantise
__device__ __forceinline__ long long mx_sf_offset(long long row, int j, int chunks_k) {
  const long long rb = row >> 7; const int rr = (int)(row & 127);
  return (rb * chunks_k + (j >> 2)) * 512 + (rr & 31) * 16 + (rr >> 5) * 4 + (j & 3);
}
__device__ __forceinline__ float e4m3_to_float(uint8_t v) {
  return __half2float(__half(__nv_cvt_fp8_to_halfraw(v, __NV_E4M3)));
}
__constant__ float MX_E2M1[8] = {0.f, 0.5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};
__device__ __forceinline__ uint32_t e2m1_code(float x) {
  const float a = fabsf(x);
  const uint32_t m = a < 0.25f ? 0u : a < 0.75f ? 1u : a < 1.25f ? 2u : a < 1.75f ? 3u : a < 2.5f ? 4u : a < 3.5f ? 5u : a < 5.f ? 6u : 7u;
  return m | (x < 0.f ? 8u : 0u);
}
template <typename T> __device__ __forceinline__ float mx_ld(const T* p);
template <> __device__ __forceinline__ float mx_ld<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float mx_ld<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }

// one thread per scale block: 32 elements (kind 0) or 16 (kind 1)
template <int KIND, typename T>
__global__ void mx_quant_kernel(const T* __restrict__ x, long long ldx, long long rows, int K, float tensor_scale,
                                uint8_t* __restrict__ data, uint8_t* __restrict__ sf) {
  constexpr int V = KIND == 0 ? 32 : 16;
  const int blocks_k = K / V, chunks_k = blocks_k / 4;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= rows * blocks_k) return;
  const long long row = idx / blocks_k; const int j = (int)(idx % blocks_k);
  const T* xp = x + row * ldx + (long long)j * V;
  float v[V];
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < V; ++i) { v[i] = mx_ld(xp + i); amax = fmaxf(amax, fabsf(v[i])); }
  if (KIND == 0) {
    int e = -127;
    if (amax > 0.f) {
      int ex; const float m = frexpf(amax / 448.f, &ex);        // amax / 448 = m * 2^ex, m in [0.5, 1)
      e = m > 0.5f ? ex : ex - 1;                                // smallest power of two that keeps the block inside e4m3
      e = max(-127, min(127, e));
    }
    sf[mx_sf_offset(row, j, chunks_k)] = (uint8_t)(e + 127);
    const float inv = ldexpf(1.f, -e);
    uint32_t w[V / 4];
#pragma unroll
    for (int i = 0; i < V; i += 4) {
      uint32_t u = 0;
#pragma unroll
      for (int b = 0; b < 4; ++b) u |= (uint32_t)__nv_cvt_float_to_fp8(v[i + b] * inv, __NV_SATFINITE, __NV_E4M3) << (8 * b);
      w[i / 4] = u;
    }
    uint4* dp = reinterpret_cast<uint4*>(data + row * (long long)K + (long long)j * V);
    dp[0] = make_uint4(w[0], w[1], w[2], w[3]);
    dp[1] = make_uint4(w[4], w[5], w[6], w[7]);
  } else {
    const uint8_t q = (uint8_t)__nv_cvt_float_to_fp8(amax / (6.f * tensor_scale), __NV_SATFINITE, __NV_E4M3);
    sf[mx_sf_offset(row, j, chunks_k)] = q;
    const float s = e4m3_to_float(q) * tensor_scale;
    const float inv = s > 0.f ? 1.f / s : 0.f;
    uint32_t w[2] = {0u, 0u};
#pragma unroll
    for (int i = 0; i < V; ++i) w[i >> 3] |= e2m1_code(v[i] * inv) << (4 * (i & 7));       // even element in the low nibble
    *reinterpret_cast<uint2*>(data + row * (long long)(K / 2) + (long long)j * (V / 2)) = make_uint2(w[0], w[1]);
  }
}

template <int KIND>
__global__ void mx_dequant_kernel(const uint8_t* __restrict__ data, const uint8_t* __restrict__ sf, long long rows, int K,
                                  float tensor_scale, float* __restrict__ out) {
  constexpr int V = KIND == 0 ? 32 : 16;
  const int blocks_k = K / V, chunks_k = blocks_k / 4;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= rows * blocks_k) return;
  const long long row = idx / blocks_k; const int j = (int)(idx % blocks_k);
  const uint8_t q = sf[mx_sf_offset(row, j, chunks_k)];
  float* op = out + row * (long long)K + (long long)j * V;
  if (KIND == 0) {
    const float s = ldexpf(1.f, (int)q - 127);
    const uint8_t* dp = data + row * (long long)K + (long long)j * V;
#pragma unroll
    for (int i = 0; i < V; ++i) op[i] = e4m3_to_float(dp[i]) * s;
  } else {
    const float s = e4m3_to_float(q) * tensor_scale;
    const uint8_t* dp = data + row * (long long)(K / 2) + (long long)j * (V / 2);
#pragma unroll
    for (int i = 0; i < V; ++i) {
      const uint32_t c = (dp[i >> 1] >> (4 * (i & 1))) & 15u;
      op[i] = (c & 8u ? -1.f : 1.f) * MX_E2M1[c & 7u] * s;
    }
  }
}

template <int KIND>
static int launch_mx(const MxGemmArgs& a, int num_sms, cudaStream_t stream) {
  using Cf = MxCfg<KIND>;
  const long long kbytes = KIND == 0 ? a.K : a.K / 2;
  CUtensorMap tmA, tmB;
  int rc = make_tmap_3d(&tmA, a.A, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, kbytes, a.M, 1, kbytes, (long long)a.M * kbytes, Cf::BKB, Cf::BM, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return 100 + rc;
  rc = make_tmap_3d(&tmB, a.B, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, kbytes, a.N, 1, kbytes, (long long)a.N * kbytes, Cf::BKB, Cf::BN, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return 200 + rc;
  const long long tiles = (long long)((a.M + Cf::BM - 1) / Cf::BM) * ((a.N + Cf::BN - 1) / Cf::BN);
  const int grid = (int)(tiles < num_sms ? tiles : num_sms);
  gemm_mx_kernel<KIND><<<grid, MX_THREADS, Cf::SMEM, stream>>>(tmA, tmB, a);
  return (int)cudaGetLastError();
}

}  // namespace b200

extern "C" int b200_gemm_mx_init() {
  using namespace b200;
  if (cudaFuncSetAttribute(gemm_mx_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, MxCfg<0>::SMEM) != cudaSuccess) return 1;
  if (cudaFuncSetAttribute(gemm_mx_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, MxCfg<1>::SMEM) != cudaSuccess) return 2;
  return 0;
}

// K must be a multiple of 128 (kind 0) or 256 (kind 1), N a multiple of 8; A, B 16-byte aligned.
extern "C" int b200_gemm_mx(const b200::MxGemmArgs* args, int num_sms, cudaStream_t stream) {
  using namespace b200;
  const MxGemmArgs& a = *args;
  if (a.M <= 0 || a.N <= 0 || a.K <= 0) return 0;
  if (a.kind != 0 && a.kind != 1) return -1;
  if (a.K % (a.kind == 0 ? 128 : 256) != 0 || a.N % 8 != 0 || a.ldc % 8 != 0) return -2;
  if ((reinterpret_cast<uintptr_t>(a.A) | reinterpret_cast<uintptr_t>(a.B) | reinterpret_cast<uintptr_t>(a.sfa) | reinterpret_cast<uintptr_t>(a.sfb) |
       reinterpret_cast<uintptr_t>(a.C)) & 15) return -3;
  return a.kind == 0 ? launch_mx<0>(a, num_sms, stream) : launch_mx<1>(a, num_sms, stream);
}

// data: [rows, K] bytes (kind 0) or [rows, K / 2] (kind 1); sf: zero-filled chunk buffer of
// ceil(rows / 256) * 2 * (K / (4 * V)) * 512 bytes (V = 32 or 16). tensor_scale is used by kind 1 only.
extern "C" int b200_mx_quant(const void* x, int is_bf16, long long ldx, long long rows, int K, int kind, float tensor_scale, void* data,
                             void* sf, cudaStream_t st) {
  using namespace b200;
  if (rows <= 0 || K <= 0) return 0;
  if (K % (kind == 0 ? 128 : 256) != 0) return -2;
  const long long n = rows * (K / (kind == 0 ? 32 : 16));
  const unsigned grid = (unsigned)((n + 127) / 128);
  if (kind == 0) {
    if (is_bf16) mx_quant_kernel<0, __nv_bfloat16><<<grid, 128, 0, st>>>((const __nv_bfloat16*)x, ldx, rows, K, tensor_scale, (uint8_t*)data, (uint8_t*)sf);
    else mx_quant_kernel<0, float><<<grid, 128, 0, st>>>((const float*)x, ldx, rows, K, tensor_scale, (uint8_t*)data, (uint8_t*)sf);
  } else {
    if (is_bf16) mx_quant_kernel<1, __nv_bfloat16><<<grid, 128, 0, st>>>((const __nv_bfloat16*)x, ldx, rows, K, tensor_scale, (uint8_t*)data, (uint8_t*)sf);
    else mx_quant_kernel<1, float><<<grid, 128, 0, st>>>((const float*)x, ldx, rows, K, tensor_scale, (uint8_t*)data, (uint8_t*)sf);
  }
  return (int)cudaGetLastError();
}

extern "C" int b200_mx_dequant(const void* data, const void* sf, long long rows, int K, int kind, float tensor_scale, float* out, cudaStream_t st) {
  using namespace b200;
  if (rows <= 0 || K <= 0) return 0;
  const long long n = rows * (K / (kind == 0 ? 32 : 16));
  const unsigned grid = (unsigned)((n + 127) / 128);
  if (kind == 0) mx_dequant_kernel<0><<<grid, 128, 0, st>>>((const uint8_t*)data, (const uint8_t*)sf, rows, K, tensor_scale, out);
  else mx_dequant_kernel<1><<<grid, 128, 0, st>>>((const uint8_t*)data, (const uint8_t*)sf, rows, K, tensor_scale, out);
  return (int)cudaGetLastError();
}
