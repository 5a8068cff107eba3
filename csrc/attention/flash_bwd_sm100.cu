// A2: FlashAttention backward on tcgen05 / TMEM (sm_100a), causal and non-causal, head_dim 64 / 128.
//
// Gradients of O = softmax(Q K^T * scale) V for an arbitrary upstream dO. (The reference's backward,
// rust-nn src/tensor.rs:1468-1554, assumes a uniform upstream gradient; the oracle here is autograd
// through dense fp32 softmax attention.)
//
// One CTA = one (batch, head, 128-key block), 128 * CG threads (CG warps per TMEM lane quarter, each owning 1/CG of
// the columns; CG = 2 measured faster than 4), looping over the query blocks that see it.
// Per query block, five tensor-core products, all operands fed from 128B-swizzled shared memory:
//   S  = Q K^T            dP = dO V^T                      (K-major x K-major)        -> TMEM
//   P  = exp2(S*c - lse)  dS = P * (dP - delta)            (tcgen05.ld, registers, bf16 tiles to smem)
//   dV += P^T dO          dK += dS^T Q                     (MN-major x MN-major, accumulate in TMEM)
//   dQ  = dS K                                             (K-major x MN-major)       -> TMEM -> fp32 atomics
// dK / dV stay resident in TMEM for the whole loop. Warp w reads TMEM lanes 32*(w%4).. (its rows) and
// the column half w/4. Every wait is bounded.
#include <type_traits>
#include "../common/ptx.cuh"
#include "../common/launch.cuh"
#include "../common/tensormap.h"
#include "flash_sm100.h"

namespace b200 {

struct BwdParams {
  __nv_bfloat16* dk; long long dk_sb, dk_ss, dk_sh;
  __nv_bfloat16* dv; long long dv_sb, dv_ss, dv_sh;
  float* dq_accum;
  const float* lse; const float* delta;
  int B, H, Sq, Skv;
  float scale, scale_log2;
  uint32_t* status;
};

// delta[b,h,s] = sum_e dO[b,s,h,e] * O[b,s,h,e]; hd/8 lanes per row, one 16-byte load of each operand per lane
__global__ void flash_delta_kernel(const __nv_bfloat16* __restrict__ o, long long o_sb, long long o_ss, long long o_sh,
                                   const __nv_bfloat16* __restrict__ d, long long d_sb, long long d_ss, long long d_sh,
                                   float* __restrict__ delta, int B, int H, int S, int hd) {
  const int lpr = hd / 8;                                   // lanes per row: 8 (hd 64) or 16 (hd 128)
  const long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  const long long w = t / lpr;
  const int sub = (int)(t % lpr);
  const long long total = (long long)B * H * S;
  float acc = 0.f;
  if (w < total) {
    // rows are enumerated [b][s][h] so that neighbouring lanes read neighbouring memory
    const int h = (int)(w % H); long long r = w / H; const int s = (int)(r % S); const int b = (int)(r / S);
    const uint4 a = __ldg(reinterpret_cast<const uint4*>(o + b * o_sb + s * o_ss + h * o_sh + sub * 8));
    const uint4 c = __ldg(reinterpret_cast<const uint4*>(d + b * d_sb + s * d_ss + h * d_sh + sub * 8));
    const float2 a0 = unpack_bf16x2(a.x), a1 = unpack_bf16x2(a.y), a2 = unpack_bf16x2(a.z), a3 = unpack_bf16x2(a.w);
    const float2 c0 = unpack_bf16x2(c.x), c1 = unpack_bf16x2(c.y), c2 = unpack_bf16x2(c.z), c3 = unpack_bf16x2(c.w);
    acc = a0.x * c0.x + a0.y * c0.y + a1.x * c1.x + a1.y * c1.y + a2.x * c2.x + a2.y * c2.y + a3.x * c3.x + a3.y * c3.y;
  }
  for (int o2 = lpr >> 1; o2; o2 >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o2);
  if (w < total && sub == 0) {
    const int h = (int)(w % H); long long r = w / H; const int s = (int)(r % S); const int b = (int)(r / S);
    delta[((long long)b * H + h) * S + s] = acc;
  }
}

// dq[b,s,h,:] (bf16, strided) = dq_accum[b,s,h,:] (fp32, contiguous)
__global__ void flash_dq_convert_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ dq, long long sb,
                                        long long ss, long long sh, int B, int S, int H, int hd) {
  pdl_trigger();
  pdl_wait();
  const long long total = (long long)B * S * H * (hd / 8);
  long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  const long long stride = (long long)gridDim.x * blockDim.x;
  const int vpr = hd / 8;
  for (; i < total; i += stride) {
    const int v = (int)(i % vpr); long long r = i / vpr;
    const int h = (int)(r % H); r /= H; const int s = (int)(r % S); const int b = (int)(r / S);
    const float4 a0 = *reinterpret_cast<const float4*>(acc + ((((long long)b * S + s) * H + h) * hd + v * 8));
    const float4 a1 = *reinterpret_cast<const float4*>(acc + ((((long long)b * S + s) * H + h) * hd + v * 8 + 4));
    uint4 o = make_uint4(pack_bf16x2(a0.x, a0.y), pack_bf16x2(a0.z, a0.w), pack_bf16x2(a1.x, a1.y), pack_bf16x2(a1.z, a1.w));
    *reinterpret_cast<uint4*>(dq + b * sb + s * ss + h * sh + v * 8) = o;
  }
}

constexpr int BWD_CG = 2;                       // column groups per row: threads = 128 * BWD_CG

template <int HD, bool CAUSAL>
__global__ void __launch_bounds__(128 * BWD_CG, 1)
flash_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO, BwdParams p) {
  constexpr int BLK = 128;
  constexpr int KA = HD / 64;
  // head_dim 64 leaves room in TMEM for a double-buffered dQ and in shared memory for three Q/dO stages: the
  // tensor cores then run dV/dK/dQ of block i and S/dP of block i+1 back to back while the CTA retires dQ of
  // block i-1. head_dim 128 fills TMEM (dK, dV 128 columns each), dQ aliases S there and the steps serialise.
  constexpr bool PIPE = (HD == 64);
  constexpr int STAGES = PIPE ? 3 : 1;
  constexpr int TILE_BYTES = BLK * HD * 2;       // one Q / dO / K / V tile
  constexpr int PS_BYTES = BLK * BLK * 2;        // P or dS tile
  constexpr uint32_t TMEM_COLS = 512;
  constexpr uint32_t COL_S = 0, COL_DP = 128, COL_DK = 256, COL_DV = 256 + HD;
  constexpr uint32_t COL_DQ = PIPE ? 384 : COL_S;   // PIPE: two buffers at 384 and 448

  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* sK = smem;
  uint8_t* sV = sK + TILE_BYTES;
  uint8_t* sQ = sV + TILE_BYTES;                 // STAGES
  uint8_t* sdO = sQ + STAGES * TILE_BYTES;       // STAGES
  uint8_t* sP = sdO + STAGES * TILE_BYTES;
  uint8_t* sdS = sP + PS_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sdS + PS_BYTES);
  uint64_t* kv_bar = bars;            // 1
  uint64_t* q_bar = bars + 1;         // up to 3 (Q and dO of one query block arrive together)
  uint64_t* sdp_bar = bars + 4;       // 1
  uint64_t* dq_bar = bars + 5;        // 1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 6);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  pdl_trigger();
  const int quarter = warp & 3, cq = warp >> 2;   // TMEM lane quarter (rows) and column group of this warp
  constexpr int CG = BWD_CG;
  constexpr int SC = 128 / CG;                    // S / dP columns per thread (32 or 64)
  constexpr int DQC = HD / CG;                    // dQ / dK / dV columns per thread (16 .. 64)
  const int row = quarter * 32 + lane;          // row of the 128-row tile this thread owns
  const int n_kv_blocks = (p.Skv + BLK - 1) / BLK;
  const int m_blocks = (p.Sq + BLK - 1) / BLK;
  int bid = blockIdx.x;
  const int jb = bid % n_kv_blocks; bid /= n_kv_blocks;   // early key blocks (most work when causal) first
  const int h = bid % p.H; const int b = bid / p.H;
  const int kv0 = jb * BLK;

  if ((smem_u32(smem) & 1023u) != 0) {
    if (tid == 0 && p.status) atomicCAS(p.status, 0u, (uint32_t)ST_BAD_ARGUMENT);
    return;
  }
  if (tid == 0) {
    mbar_init(kv_bar, 1);
    for (int s = 0; s < STAGES; ++s) mbar_init(&q_bar[s], 1);
    mbar_init(sdp_bar, 1); mbar_init(dq_bar, 1);
    fence_barrier_init();
    tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV); tma_prefetch_desc(&tmdO);
  }
  if (warp == 0) { tmem_alloc(tmem_slot, TMEM_COLS); tmem_relinquish(); }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_row = tmem_base + (uint32_t(quarter * 32) << 16);
  pdl_wait();

  const int i_start = CAUSAL ? (kv0 / BLK) : 0;
  const int n_iter = m_blocks - i_start;

  constexpr uint32_t idesc_kk = make_idesc(BLK, BLK, CFMT_F32, FMT_BF16, FMT_BF16, 0, 0);   // S, dP
  constexpr uint32_t idesc_mm = make_idesc(BLK, HD, CFMT_F32, FMT_BF16, FMT_BF16, 1, 1);    // dV, dK
  constexpr uint32_t idesc_km = make_idesc(BLK, HD, CFMT_F32, FMT_BF16, FMT_BF16, 0, 1);    // dQ

  auto load_q = [&](int it) {
    const int st = it % STAGES; const int i = i_start + it;
    mbar_expect_tx(&q_bar[st], 2 * TILE_BYTES);
#pragma unroll
    for (int a = 0; a < KA; ++a) {
      tma_load_4d(sQ + st * TILE_BYTES + a * (BLK * 128), &tmQ, &q_bar[st], a * 64, h, i * BLK, b);
      tma_load_4d(sdO + st * TILE_BYTES + a * (BLK * 128), &tmdO, &q_bar[st], a * 64, h, i * BLK, b);
    }
  };
  // MMA issue is a single thread's serial instruction stream on the critical path: descriptors are a base word
  // plus an immediate, accumulate flags are compile-time.
  auto issue_s_dp = [&](int it) {
    const int st = it % STAGES;
    const uint32_t lQ = sdesc_lo(smem_u32(sQ + st * TILE_BYTES), 0), ldO = sdesc_lo(smem_u32(sdO + st * TILE_BYTES), 0);
    const uint32_t lK = sdesc_lo(smem_u32(sK), 0), lV = sdesc_lo(smem_u32(sV), 0);
#pragma unroll
    for (int k = 0; k < HD / 16; ++k) {
      const uint32_t adv = (k >> 2) * (BLK * 128) + (k & 3) * 32;
      if (k == 0) umma_f16_c<false>(tmem_base + COL_S, sdesc_at<1024>(lQ, adv), sdesc_at<1024>(lK, adv), idesc_kk);
      else umma_f16_c<true>(tmem_base + COL_S, sdesc_at<1024>(lQ, adv), sdesc_at<1024>(lK, adv), idesc_kk);
    }
#pragma unroll
    for (int k = 0; k < HD / 16; ++k) {
      const uint32_t adv = (k >> 2) * (BLK * 128) + (k & 3) * 32;
      if (k == 0) umma_f16_c<false>(tmem_base + COL_DP, sdesc_at<1024>(ldO, adv), sdesc_at<1024>(lV, adv), idesc_kk);
      else umma_f16_c<true>(tmem_base + COL_DP, sdesc_at<1024>(ldO, adv), sdesc_at<1024>(lV, adv), idesc_kk);
    }
    tc_commit(sdp_bar);
  };
  auto issue_grads = [&](int it, bool commit) {
    const int st = it % STAGES;
    // MN-major views (dV, dK operands): atoms of 64 rows BLK*128 bytes apart
    const uint32_t mQ = sdesc_lo(smem_u32(sQ + st * TILE_BYTES), BLK * 128), mdO = sdesc_lo(smem_u32(sdO + st * TILE_BYTES), BLK * 128);
    const uint32_t mP = sdesc_lo(smem_u32(sP), BLK * 128), mdS = sdesc_lo(smem_u32(sdS), BLK * 128), mK = sdesc_lo(smem_u32(sK), BLK * 128);
    const uint32_t kdS = sdesc_lo(smem_u32(sdS), 0);                       // K-major view of dS (dQ's A operand)
    const uint32_t dq_col = PIPE ? COL_DQ + (uint32_t)(it & 1) * 64u : COL_DQ;
    const bool acc0 = it > 0;
#pragma unroll
    for (int k = 0; k < BLK / 16; ++k) {   // dV += P^T dO   (K dimension = query rows)
      if (k == 0 && !acc0) umma_f16_c<false>(tmem_base + COL_DV, sdesc_at<1024>(mP, 0), sdesc_at<1024>(mdO, 0), idesc_mm);
      else umma_f16_c<true>(tmem_base + COL_DV, sdesc_at<1024>(mP, k * 2048), sdesc_at<1024>(mdO, k * 2048), idesc_mm);
    }
#pragma unroll
    for (int k = 0; k < BLK / 16; ++k) {   // dK += dS^T Q
      if (k == 0 && !acc0) umma_f16_c<false>(tmem_base + COL_DK, sdesc_at<1024>(mdS, 0), sdesc_at<1024>(mQ, 0), idesc_mm);
      else umma_f16_c<true>(tmem_base + COL_DK, sdesc_at<1024>(mdS, k * 2048), sdesc_at<1024>(mQ, k * 2048), idesc_mm);
    }
#pragma unroll
    for (int k = 0; k < BLK / 16; ++k) {   // dQ = dS K      (K dimension = key rows)
      const uint32_t adv = (k >> 2) * (BLK * 128) + (k & 3) * 32;
      if (k == 0) umma_f16_c<false>(tmem_base + dq_col, sdesc_at<1024>(kdS, adv), sdesc_at<1024>(mK, k * 2048), idesc_km);
      else umma_f16_c<true>(tmem_base + dq_col, sdesc_at<1024>(kdS, adv), sdesc_at<1024>(mK, k * 2048), idesc_km);
    }
    if (commit) tc_commit(dq_bar);
  };
  // dQ rows of query block `it` -> fp32 atomics (scaled). The block's MMAs must be known complete.
  auto retire_dq = [&](int it) {
    const int q_row = (i_start + it) * BLK + row;
    const uint32_t dq_col = PIPE ? COL_DQ + (uint32_t)(it & 1) * 64u : COL_DQ;
    float* dst = p.dq_accum + ((((long long)b * p.Sq + q_row) * p.H + h) * HD) + cq * DQC;
    uint32_t v[DQC];
    if constexpr (DQC == 16) tmem_ld_x16(tmem_row + dq_col + cq * DQC, v);
    else {
#pragma unroll
      for (int c = 0; c < DQC / 32; ++c) tmem_ld_x32(tmem_row + dq_col + cq * DQC + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&v[c * 32]));
    }
    tmem_ld_wait();
    if (q_row < p.Sq) {
#pragma unroll
      for (int e = 0; e < DQC; e += 4) {
        float4 a = make_float4(__uint_as_float(v[e]) * p.scale, __uint_as_float(v[e + 1]) * p.scale,
                               __uint_as_float(v[e + 2]) * p.scale, __uint_as_float(v[e + 3]) * p.scale);
        atomicAdd(reinterpret_cast<float4*>(dst + e), a);
      }
    }
  };
  // P = exp2(S c - lse), dS = P (dP - delta) for this thread's row and column half -> bf16 tiles in shared memory
  auto softmax_block = [&](auto masked, int q_row, bool row_ok, float lse2, float dlt) {
    constexpr bool MASK = decltype(masked)::value;
    const int col0 = cq * SC;                    // this thread's SC key columns
    // every TMEM load of the thread goes out before the single wait: one exposed latency
    uint32_t sv[SC], dv[SC];
#pragma unroll
    for (int c = 0; c < SC / 32; ++c) {
      tmem_ld_x32(tmem_row + COL_S + col0 + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&sv[c * 32]));
      tmem_ld_x32(tmem_row + COL_DP + col0 + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&dv[c * 32]));
    }
    tmem_ld_wait();
#pragma unroll
    for (int g = 0; g < SC / 8; ++g) {
      float pp[8], ds[8];
      // packed fp32 pairs for the exponent argument, dP - delta and the product: this loop is bound by instruction issue
#pragma unroll
      for (int u = 0; u < 8; u += 2) {
        const int e = g * 8 + u;
        float a0 = __uint_as_float(sv[e]), a1 = __uint_as_float(sv[e + 1]);
        fma2_scalar(a0, a1, p.scale_log2, -lse2);
        float p0 = ex2_approx(a0), p1 = ex2_approx(a1);
        if (MASK) {
          if (!row_ok || (CAUSAL && (kv0 + col0 + e > q_row))) p0 = 0.f;
          if (!row_ok || (CAUSAL && (kv0 + col0 + e + 1 > q_row))) p1 = 0.f;
        }
        float d0 = __uint_as_float(dv[e]), d1 = __uint_as_float(dv[e + 1]);
        add2(d0, d1, -dlt, -dlt);
        mul2(d0, d1, p0, p1);
        pp[u] = p0; pp[u + 1] = p1; ds[u] = d0; ds[u + 1] = d1;
      }
      const int cc = (col0 >> 3) + g;
      const int atom = cc >> 3, chunk = cc & 7;
      const uint32_t off = atom * (BLK * 128) + sw128_offset(row, chunk);
      *reinterpret_cast<uint4*>(sP + off) = make_uint4(pack_bf16x2(pp[0], pp[1]), pack_bf16x2(pp[2], pp[3]), pack_bf16x2(pp[4], pp[5]), pack_bf16x2(pp[6], pp[7]));
      *reinterpret_cast<uint4*>(sdS + off) = make_uint4(pack_bf16x2(ds[0], ds[1]), pack_bf16x2(ds[2], ds[3]), pack_bf16x2(ds[4], ds[5]), pack_bf16x2(ds[6], ds[7]));
    }
  };

  bool ok = true;
  if (tid == 0 && n_iter > 0) {
    mbar_expect_tx(kv_bar, 2 * TILE_BYTES);
#pragma unroll
    for (int a = 0; a < KA; ++a) {
      tma_load_4d(sK + a * (BLK * 128), &tmK, kv_bar, a * 64, h, kv0, b);
      tma_load_4d(sV + a * (BLK * 128), &tmV, kv_bar, a * 64, h, kv0, b);
    }
    for (int s = 0; s < STAGES && s < n_iter; ++s) load_q(s);
    ok = mbar_wait(kv_bar, 0, p.status, ST_TIMEOUT_TMA_FULL) && mbar_wait(&q_bar[0], 0, p.status, ST_TIMEOUT_TMA_FULL);
    if (ok) { tc_fence_after_sync(); issue_s_dp(0); }
  }

  const float log2e = 1.4426950408889634f;
  // per-row statistics of the next query block are fetched one iteration ahead (their latency hides behind the MMAs)
  auto load_stats = [&](int it, float& lse2, float& dlt) {
    const int q_row = (i_start + it) * BLK + row;
    if (it < n_iter && q_row < p.Sq) {
      const long long idx = ((long long)b * p.H + h) * p.Sq + q_row;
      lse2 = __ldg(p.lse + idx) * log2e; dlt = __ldg(p.delta + idx);
    } else { lse2 = 0.f; dlt = 0.f; }
  };
  float lse2_n, dlt_n;
  load_stats(0, lse2_n, dlt_n);

  for (int it = 0; it < n_iter; ++it) {
    const int q0 = (i_start + it) * BLK;
    const int q_row = q0 + row;
    const bool row_ok = q_row < p.Sq;
    const float lse2 = lse2_n, dlt = dlt_n;
    load_stats(it + 1, lse2_n, dlt_n);
    if (!mbar_wait(sdp_bar, it & 1, p.status, ST_TIMEOUT_ACC_FULL)) ok = false;      // S/dP of block it (and every MMA before) done
    if (__syncthreads_or(!ok)) { ok = false; break; }
    tc_fence_after_sync();
    const bool need_mask = (CAUSAL && (kv0 + BLK - 1 > q0)) || (q0 + BLK > p.Sq);
    if (need_mask) softmax_block(std::true_type{}, q_row, row_ok, lse2, dlt);
    else softmax_block(std::false_type{}, q_row, row_ok, lse2, dlt);
    tc_fence_before_sync();
    fence_proxy_async_smem();
    __syncthreads();
    if constexpr (PIPE) {
      if (tid == 0) {
        tc_fence_after_sync();
        const bool last = (it + 1 == n_iter);
        issue_grads(it, last);
        if (!last) {
          ok = mbar_wait(&q_bar[(it + 1) % STAGES], ((it + 1) / STAGES) & 1, p.status, ST_TIMEOUT_TMA_FULL);
          if (ok) { tc_fence_after_sync(); issue_s_dp(it + 1); }
        }
      }
      // while the tensor cores work: retire dQ of the previous block (complete since this iteration's sdp_bar)
      if (it > 0) {
        retire_dq(it - 1);
        // Q/dO stage of block it-1 is free as well
        if (tid == 0 && it - 1 + STAGES < n_iter) load_q(it - 1 + STAGES);
      }
      tc_fence_before_sync();
    } else {
      if (tid == 0) { tc_fence_after_sync(); issue_grads(it, true); }
      if (!mbar_wait(dq_bar, it & 1, p.status, ST_TIMEOUT_ACC_FULL)) ok = false;
      if (__syncthreads_or(!ok)) { ok = false; break; }
      tc_fence_after_sync();
      if (tid == 0 && it + STAGES < n_iter) load_q(it + STAGES);
      retire_dq(it);
      tc_fence_before_sync();
      __syncthreads();
      if (tid == 0 && it + 1 < n_iter) {
        ok = mbar_wait(&q_bar[(it + 1) % STAGES], ((it + 1) / STAGES) & 1, p.status, ST_TIMEOUT_TMA_FULL);
        if (ok) { tc_fence_after_sync(); issue_s_dp(it + 1); }
      }
    }
  }
  if constexpr (PIPE) {
    if (n_iter > 0) {
      if (ok && !mbar_wait(dq_bar, 0, p.status, ST_TIMEOUT_ACC_FULL)) ok = false;      // the last block's dV / dK / dQ
      if (__syncthreads_or(!ok)) ok = false;
      if (ok) { tc_fence_after_sync(); retire_dq(n_iter - 1); }
    }
  }

  // dK / dV: TMEM -> bf16 global. Thread owns key row `row`, column quarter `cq`.
  if (ok && n_iter > 0) {
    tc_fence_after_sync();
    const int kv_row = kv0 + row;
    const int colbase = cq * DQC;
    uint32_t vk[DQC], vv[DQC];
    if constexpr (DQC == 16) { tmem_ld_x16(tmem_row + COL_DK + colbase, vk); tmem_ld_x16(tmem_row + COL_DV + colbase, vv); }
    else {
#pragma unroll
      for (int c = 0; c < DQC / 32; ++c) {
        tmem_ld_x32(tmem_row + COL_DK + colbase + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&vk[c * 32]));
        tmem_ld_x32(tmem_row + COL_DV + colbase + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&vv[c * 32]));
      }
    }
    tmem_ld_wait();
    if (kv_row < p.Skv) {
      __nv_bfloat16* dkp = p.dk + (long long)b * p.dk_sb + (long long)kv_row * p.dk_ss + (long long)h * p.dk_sh + colbase;
      __nv_bfloat16* dvp = p.dv + (long long)b * p.dv_sb + (long long)kv_row * p.dv_ss + (long long)h * p.dv_sh + colbase;
#pragma unroll
      for (int e = 0; e < DQC; e += 8) {
        *reinterpret_cast<uint4*>(dkp + e) = make_uint4(
            pack_bf16x2(__uint_as_float(vk[e]) * p.scale, __uint_as_float(vk[e + 1]) * p.scale),
            pack_bf16x2(__uint_as_float(vk[e + 2]) * p.scale, __uint_as_float(vk[e + 3]) * p.scale),
            pack_bf16x2(__uint_as_float(vk[e + 4]) * p.scale, __uint_as_float(vk[e + 5]) * p.scale),
            pack_bf16x2(__uint_as_float(vk[e + 6]) * p.scale, __uint_as_float(vk[e + 7]) * p.scale));
        *reinterpret_cast<uint4*>(dvp + e) = make_uint4(
            pack_bf16x2(__uint_as_float(vv[e]), __uint_as_float(vv[e + 1])), pack_bf16x2(__uint_as_float(vv[e + 2]), __uint_as_float(vv[e + 3])),
            pack_bf16x2(__uint_as_float(vv[e + 4]), __uint_as_float(vv[e + 5])), pack_bf16x2(__uint_as_float(vv[e + 6]), __uint_as_float(vv[e + 7])));
      }
    }
  } else if (ok && n_iter <= 0) {
    // a key block no query attends to (cannot happen for causal self-attention): zero gradients
    const int kv_row = kv0 + row;
    if (kv_row < p.Skv) {
      for (int e = cq * DQC; e < (cq + 1) * DQC; ++e) {
        p.dk[(long long)b * p.dk_sb + (long long)kv_row * p.dk_ss + (long long)h * p.dk_sh + e] = __float2bfloat16(0.f);
        p.dv[(long long)b * p.dv_sb + (long long)kv_row * p.dv_ss + (long long)h * p.dv_sh + e] = __float2bfloat16(0.f);
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) { tc_fence_after_sync(); tmem_dealloc(tmem_base, TMEM_COLS); }
}

template <int HD, bool CAUSAL>
static int bwd_set_attr() {
  static bool done = false;
  if (done) return 0;
  constexpr int STAGES = (HD == 64) ? 3 : 1;
  constexpr int SMEM = 2 * 128 * HD * 2 + 2 * STAGES * 128 * HD * 2 + 2 * 128 * 128 * 2 + 128;
  (void)cudaGetLastError();
  if (cudaFuncSetAttribute(flash_bwd_kernel<HD, CAUSAL>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess) return 1;
  done = true;
  return 0;
}

template <int HD, bool CAUSAL>
static int launch_bwd(const FlashArgs& a, cudaStream_t st) {
  CUtensorMap tmQ, tmK, tmV, tmdO;
  const auto BF = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const auto SW = CU_TENSOR_MAP_SWIZZLE_128B;
  if (make_tmap_attn(&tmQ, a.q.ptr, BF, 2, a.hd, a.H, a.Sq, a.B, a.q.sh, a.q.ss, a.q.sb, 64, 128, SW)) return 101;
  if (make_tmap_attn(&tmK, a.k.ptr, BF, 2, a.hd, a.H, a.Skv, a.B, a.k.sh, a.k.ss, a.k.sb, 64, 128, SW)) return 102;
  if (make_tmap_attn(&tmV, a.v.ptr, BF, 2, a.hd, a.H, a.Skv, a.B, a.v.sh, a.v.ss, a.v.sb, 64, 128, SW)) return 103;
  if (make_tmap_attn(&tmdO, a.dout.ptr, BF, 2, a.hd, a.H, a.Sq, a.B, a.dout.sh, a.dout.ss, a.dout.sb, 64, 128, SW)) return 104;
  constexpr int STAGES = (HD == 64) ? 3 : 1;
  constexpr int SMEM = 2 * 128 * HD * 2 + 2 * STAGES * 128 * HD * 2 + 2 * 128 * 128 * 2 + 128;
  auto kfn = flash_bwd_kernel<HD, CAUSAL>;
  if (bwd_set_attr<HD, CAUSAL>()) return 105;
  const long long rows = (long long)a.B * a.H * a.Sq;
  flash_delta_kernel<<<(unsigned)((rows * (a.hd / 8) + 255) / 256), 256, 0, st>>>(
      (const __nv_bfloat16*)a.o.ptr, a.o.sb, a.o.ss, a.o.sh, (const __nv_bfloat16*)a.dout.ptr, a.dout.sb, a.dout.ss,
      a.dout.sh, a.delta, a.B, a.H, a.Sq, a.hd);
  cudaMemsetAsync(a.dq_accum, 0, sizeof(float) * (size_t)a.B * a.Sq * a.H * a.hd, st);
  BwdParams p;
  p.dk = (__nv_bfloat16*)a.dk.ptr; p.dk_sb = a.dk.sb; p.dk_ss = a.dk.ss; p.dk_sh = a.dk.sh;
  p.dv = (__nv_bfloat16*)a.dv.ptr; p.dv_sb = a.dv.sb; p.dv_ss = a.dv.ss; p.dv_sh = a.dv.sh;
  p.dq_accum = a.dq_accum; p.lse = a.lse; p.delta = a.delta;
  p.B = a.B; p.H = a.H; p.Sq = a.Sq; p.Skv = a.Skv;
  p.scale = a.scale; p.scale_log2 = a.scale * 1.4426950408889634f; p.status = a.status;
  const long long grid = (long long)((a.Skv + 127) / 128) * a.H * a.B;
  launch_pdl(kfn, dim3((unsigned)grid), dim3(128 * BWD_CG), SMEM, st, tmQ, tmK, tmV, tmdO, p);
  long long total = (long long)a.B * a.Sq * a.H * (a.hd / 8);
  long long g = (total + 255) / 256; if (g > 148 * 16) g = 148 * 16;
  launch_pdl(flash_dq_convert_kernel, dim3((unsigned)g), dim3(256), 0, st, (const float*)a.dq_accum, (__nv_bfloat16*)a.dq.ptr, a.dq.sb, a.dq.ss, a.dq.sh,
             a.B, a.Sq, a.H, a.hd);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}

}  // namespace b200

extern "C" int b200_flash_bwd_init() {
  using namespace b200;
  return bwd_set_attr<64, true>() | bwd_set_attr<64, false>() | bwd_set_attr<128, true>() | bwd_set_attr<128, false>();
}

extern "C" int b200_flash_bwd(const b200::FlashArgs* a, cudaStream_t st) {
  using namespace b200;
  if (a->B <= 0 || a->H <= 0 || a->Sq <= 0 || a->Skv <= 0) return 0;
  if (a->hd == 64) return a->causal ? launch_bwd<64, true>(*a, st) : launch_bwd<64, false>(*a, st);
  if (a->hd == 128) return a->causal ? launch_bwd<128, true>(*a, st) : launch_bwd<128, false>(*a, st);
  return -3;
}
