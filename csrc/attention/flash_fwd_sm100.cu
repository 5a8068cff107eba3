// A1: FlashAttention forward on tcgen05 / TMEM (sm_100a), causal and non-causal, head_dim 64 / 128.
//
// Exact softmax(Q K^T * scale) V with an online softmax; the oracle is dense fp32 softmax attention,
// the same mathematics as rust-nn src/tensor.rs:618-677 and its WGSL shader src/gpu.rs:95-133
// (which stream keys per query on scalar units).
//
// One CTA = one (batch, head, 128-query block); 128 threads; thread t owns query row t = TMEM lane t.
//   S  = Q K_j^T     tcgen05.mma, both operands K-major 128B-swizzled tiles written by TMA   -> TMEM
//   P  = exp2(S*c - m)  read back with tcgen05.ld (one row per thread: no shuffles), written to
//                        shared memory as a bf16 K-major swizzled A operand
//   O += P V_j       tcgen05.mma accumulating in TMEM, V consumed MN-major straight from its [kv][hd] layout;
//                    O is rescaled (TMEM load / store) only when the running maximum grows by > 2^8
// S_{j+1} is issued right behind P V_j, K/V tiles are double-buffered by TMA, and two CTAs share an SM
// (TMEM 2 x 256 columns) so one CTA's exponentials overlap the other's MMAs. Every wait is bounded.
#include "../common/ptx.cuh"
#include "../common/launch.cuh"
#include "../common/tensormap.h"
#include "flash_sm100.h"

namespace b200 {

struct FwdParams {
  __nv_bfloat16* o; long long o_sb, o_ss, o_sh;
  float* lse;
  int B, H, Sq, Skv;
  float scale_log2;
  uint32_t* status;
  int global_order;      // causal: schedule ALL heads' heaviest query blocks first (only while K and V of all heads fit L2-ish)
};

template <int HD, int BN, bool CAUSAL>
__global__ void __launch_bounds__(128, 2)
flash_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, FwdParams p) {
  constexpr int BMQ = 128;
  constexpr int KA = HD / 64;                 // 64-element atoms along head_dim
  constexpr int Q_BYTES = BMQ * HD * 2;
  constexpr int KV_BYTES = BN * HD * 2;
  constexpr int P_BYTES = BMQ * BN * 2;
  constexpr uint32_t TMEM_COLS = 256;
  constexpr uint32_t PV_COL = 128;

  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + Q_BYTES;                 // 2 stages
  uint8_t* sV = sK + 2 * KV_BYTES;            // 2 stages
  uint8_t* sP = sV + 2 * KV_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + P_BYTES);
  uint64_t* q_bar = bars;          // 1
  uint64_t* k_bar = bars + 1;      // 2
  uint64_t* v_bar = bars + 3;      // 2
  uint64_t* s_bar = bars + 5;      // 1
  uint64_t* pv_bar = bars + 6;     // 1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 7);

  const int tid = threadIdx.x, warp = tid >> 5;
  pdl_trigger();
  const int m_blocks = (p.Sq + BMQ - 1) / BMQ;
  int bid = blockIdx.x;
  // heavy (late, causal) query blocks first
  const int n_bh = p.B * p.H;
  // heavy (late, causal) query blocks first: across all heads when their K / V stay cache-resident (the last wave is
  // then made of the lightest CTAs), else per head (CTAs of one head run together and share its K / V in L2)
  const bool glob = CAUSAL && p.global_order;
  const int qb = glob ? m_blocks - 1 - bid / n_bh : m_blocks - 1 - (bid % m_blocks);
  bid = glob ? bid % n_bh : bid / m_blocks;
  const int h = bid % p.H; const int b = bid / p.H;
  const int q0 = qb * BMQ;

  if ((smem_u32(smem) & 1023u) != 0) {          // swizzled tiles need 1024-byte alignment
    if (tid == 0 && p.status) atomicCAS(p.status, 0u, (uint32_t)ST_BAD_ARGUMENT);
    return;
  }
  if (tid == 0) {
    mbar_init(q_bar, 1);
    mbar_init(&k_bar[0], 1); mbar_init(&k_bar[1], 1);
    mbar_init(&v_bar[0], 1); mbar_init(&v_bar[1], 1);
    mbar_init(s_bar, 1); mbar_init(pv_bar, 1);
    fence_barrier_init();
    tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
  }
  if (warp == 0) { tmem_alloc(tmem_slot, TMEM_COLS); tmem_relinquish(); }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_row = tmem_base + (uint32_t(warp * 32) << 16);
  pdl_wait();

  int n_blocks = (p.Skv + BN - 1) / BN;
  if (CAUSAL) { int lim = (q0 + BMQ + BN - 1) / BN; if (lim < n_blocks) n_blocks = lim; }

  constexpr uint32_t idesc_s = make_idesc(BMQ, BN, CFMT_F32, FMT_BF16, FMT_BF16, 0, 0);
  constexpr uint32_t idesc_pv = make_idesc(BMQ, HD, CFMT_F32, FMT_BF16, FMT_BF16, 0, 1);

  auto load_k = [&](int j) {
    const int st = j & 1;
    mbar_expect_tx(&k_bar[st], KV_BYTES);
#pragma unroll
    for (int a = 0; a < KA; ++a) tma_load_4d(sK + st * KV_BYTES + a * (BN * 128), &tmK, &k_bar[st], a * 64, h, j * BN, b);
  };
  auto load_v = [&](int j) {
    const int st = j & 1;
    mbar_expect_tx(&v_bar[st], KV_BYTES);
#pragma unroll
    for (int a = 0; a < KA; ++a) tma_load_4d(sV + st * KV_BYTES + a * (BN * 128), &tmV, &v_bar[st], a * 64, h, j * BN, b);
  };
  // MMA issue is one thread's serial instruction stream on the critical path: descriptors are a base word plus
  // an immediate, accumulate flags are compile-time.
  auto issue_s = [&](int j) {   // S = Q K_j^T
    const int st = j & 1;
    const uint32_t lQ = sdesc_lo(smem_u32(sQ), 0), lK = sdesc_lo(smem_u32(sK + st * KV_BYTES), 0);
#pragma unroll
    for (int k = 0; k < HD / 16; ++k) {
      const uint32_t advq = (k >> 2) * (BMQ * 128) + (k & 3) * 32, advk = (k >> 2) * (BN * 128) + (k & 3) * 32;
      if (k == 0) umma_f16_c<false>(tmem_base, sdesc_at<1024>(lQ, advq), sdesc_at<1024>(lK, advk), idesc_s);
      else umma_f16_c<true>(tmem_base, sdesc_at<1024>(lQ, advq), sdesc_at<1024>(lK, advk), idesc_s);
    }
    tc_commit(s_bar);
  };
  auto issue_pv = [&](int j) {  // O (+)= P V_j
    const int st = j & 1;
    const uint32_t lP = sdesc_lo(smem_u32(sP), 0), mV = sdesc_lo(smem_u32(sV + st * KV_BYTES), BN * 128);
#pragma unroll
    for (int k = 0; k < BN / 16; ++k) {
      const uint32_t advp = (k >> 2) * (BMQ * 128) + (k & 3) * 32;
      if (k == 0 && j == 0) umma_f16_c<false>(tmem_base + PV_COL, sdesc_at<1024>(lP, 0), sdesc_at<1024>(mV, 0), idesc_pv);
      else umma_f16_c<true>(tmem_base + PV_COL, sdesc_at<1024>(lP, advp), sdesc_at<1024>(mV, k * 2048), idesc_pv);
    }
    tc_commit(pv_bar);
  };

  bool ok = true;
  if (tid == 0) {
    mbar_expect_tx(q_bar, Q_BYTES);
#pragma unroll
    for (int a = 0; a < KA; ++a) tma_load_4d(sQ + a * (BMQ * 128), &tmQ, q_bar, a * 64, h, q0, b);
    load_k(0); load_v(0);
    if (n_blocks > 1) { load_k(1); load_v(1); }
    ok = mbar_wait(q_bar, 0, p.status, ST_TIMEOUT_TMA_FULL) && mbar_wait(&k_bar[0], 0, p.status, ST_TIMEOUT_TMA_FULL);
    if (ok) { tc_fence_after_sync(); issue_s(0); }
  }

  // Online softmax with the output accumulator RESIDENT IN TMEM: P V_j accumulates onto O on the tensor
  // cores and O is only touched by threads when the running maximum grows by more than 2^8 (lazy
  // rescaling; P stays below 2^8, exact after the final division by l, which uses the same reference).
  // m_used: the maximum the exponentials currently refer to (log2 domain); l_run: row sum in that scale.
  float m_used = -INFINITY, l_run = 0.f;
  const int q_row = q0 + tid;
  const float c = p.scale_log2;

  for (int j = 0; j < n_blocks; ++j) {
    const int st = j & 1;
    if (!mbar_wait(s_bar, j & 1, p.status, ST_TIMEOUT_ACC_FULL)) { ok = false; }      // S_j done, and with it P V_{j-1}
    if (__syncthreads_or(!ok)) { ok = false; break; }
    tc_fence_after_sync();
    // K_j has been consumed by S_j and V_{j-1} by P V_{j-1}: refill those buffers (K two blocks ahead, V one)
    if (tid == 0) {
      if (j + 2 < n_blocks) load_k(j + 2);
      if (j >= 1 && j + 1 < n_blocks) load_v(j + 1);
    }
    const int kv0 = j * BN;
    const bool need_mask = (kv0 + BN > p.Skv) || (CAUSAL && (kv0 + BN - 1 > q0));
    // the whole row of S in registers: one pass over TMEM
    float s[BN];
#pragma unroll
    for (int cc = 0; cc < BN / 32; ++cc) tmem_ld_x32(tmem_row + cc * 32, *reinterpret_cast<uint32_t(*)[32]>(&s[cc * 32]));
    tmem_ld_wait();
    if (need_mask) {
#pragma unroll
      for (int i = 0; i < BN; ++i) {
        const int col = kv0 + i;
        if (col >= p.Skv || (CAUSAL && col > q_row)) s[i] = -INFINITY;
      }
    }
    // four independent chains of 3-input maxima: a 128-long dependent chain would cost its latency 128 times over
    float mx0 = s[0], mx1 = s[1], mx2 = s[2], mx3 = s[3];
#pragma unroll
    for (int i = 4; i + 8 <= BN - 4; i += 8) {
      mx0 = max3(mx0, s[i], s[i + 4]); mx1 = max3(mx1, s[i + 1], s[i + 5]);
      mx2 = max3(mx2, s[i + 2], s[i + 6]); mx3 = max3(mx3, s[i + 3], s[i + 7]);
    }
    { mx0 = fmaxf(mx0, s[BN - 4]); mx1 = fmaxf(mx1, s[BN - 3]); mx2 = fmaxf(mx2, s[BN - 2]); mx3 = fmaxf(mx3, s[BN - 1]); }
    const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
    const float m_new = fmaxf(m_used, mx * c);
    const bool grow = m_new > m_used + 8.f;                     // also true on the first finite maximum (m_used = -inf)
    if (__any_sync(0xffffffffu, grow)) {                        // TMEM accesses are warp-wide: the warp rescales together
      const float alpha = (m_new == -INFINITY) ? 1.f : ex2_approx(m_used - m_new);
      if (j > 0) {
#pragma unroll
        for (int cc = 0; cc < HD / 32; ++cc) {
          uint32_t o[32];
          tmem_ld_x32(tmem_row + PV_COL + cc * 32, o);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tmem_st_x32(tmem_row + PV_COL + cc * 32, o);
        }
        tmem_st_wait();
      }
      l_run *= alpha;
      m_used = m_new;
    }
    const float m_ref = (m_used == -INFINITY) ? 0.f : m_used;
    // exponent arguments and row sums as packed fp32 pairs: half the FMA / ADD instructions of the scalar form
    float rs0 = 0.f, rs1 = 0.f, rs2 = 0.f, rs3 = 0.f;
    const float neg_m = -m_ref;
#pragma unroll
    for (int i = 0; i < BN; i += 4) {
      fma2_scalar(s[i], s[i + 1], c, neg_m);
      fma2_scalar(s[i + 2], s[i + 3], c, neg_m);
      s[i] = ex2_approx(s[i]); s[i + 1] = ex2_approx(s[i + 1]); s[i + 2] = ex2_approx(s[i + 2]); s[i + 3] = ex2_approx(s[i + 3]);
      add2(rs0, rs1, s[i], s[i + 1]);
      add2(rs2, rs3, s[i + 2], s[i + 3]);
    }
    l_run += (rs0 + rs1) + (rs2 + rs3);
    // bf16 P tile into shared memory (K-major, 128B swizzle)
#pragma unroll
    for (int g = 0; g < BN / 8; ++g) {
      const int atom = g >> 3, chunk = g & 7;
      uint4 o = make_uint4(pack_bf16x2(s[g * 8 + 0], s[g * 8 + 1]), pack_bf16x2(s[g * 8 + 2], s[g * 8 + 3]),
                           pack_bf16x2(s[g * 8 + 4], s[g * 8 + 5]), pack_bf16x2(s[g * 8 + 6], s[g * 8 + 7]));
      *reinterpret_cast<uint4*>(sP + atom * (BMQ * 128) + sw128_offset(tid, chunk)) = o;
    }
    tc_fence_before_sync();
    fence_proxy_async_smem();
    __syncthreads();
    if (tid == 0) {
      ok = mbar_wait(&v_bar[st], (j >> 1) & 1, p.status, ST_TIMEOUT_TMA_FULL);
      if (ok) {
        tc_fence_after_sync();
        issue_pv(j);                                              // O (+)= P V_j ; commits pv_bar
        if (j + 1 < n_blocks) {
          ok = mbar_wait(&k_bar[st ^ 1], ((j + 1) >> 1) & 1, p.status, ST_TIMEOUT_TMA_FULL);
          if (ok) issue_s(j + 1);
        }
      }
    }
  }
  // the last P V: wait for its commit (pv_bar completes once per block; parity of the last one)
  if (ok && !mbar_wait(pv_bar, (n_blocks - 1) & 1, p.status, ST_TIMEOUT_ACC_FULL)) ok = false;
  if (__syncthreads_or(!ok)) ok = false;
  tc_fence_after_sync();

  if (ok) {
    const float inv_l = l_run > 0.f ? 1.f / l_run : 0.f;
    __nv_bfloat16* op = p.o + (long long)b * p.o_sb + (long long)q_row * p.o_ss + (long long)h * p.o_sh;
#pragma unroll
    for (int cc = 0; cc < HD / 32; ++cc) {
      uint32_t v[32];
      tmem_ld_x32(tmem_row + PV_COL + cc * 32, v);
      tmem_ld_wait();
      if (q_row < p.Sq) {
#pragma unroll
        for (int i = 0; i < 32; i += 8) {
          uint4 o = make_uint4(pack_bf16x2(__uint_as_float(v[i]) * inv_l, __uint_as_float(v[i + 1]) * inv_l),
                               pack_bf16x2(__uint_as_float(v[i + 2]) * inv_l, __uint_as_float(v[i + 3]) * inv_l),
                               pack_bf16x2(__uint_as_float(v[i + 4]) * inv_l, __uint_as_float(v[i + 5]) * inv_l),
                               pack_bf16x2(__uint_as_float(v[i + 6]) * inv_l, __uint_as_float(v[i + 7]) * inv_l));
          *reinterpret_cast<uint4*>(op + cc * 32 + i) = o;
        }
      }
    }
    if (p.lse && q_row < p.Sq) {
      const float mu = (m_used == -INFINITY) ? 0.f : m_used;
      p.lse[((long long)b * p.H + h) * p.Sq + q_row] = (mu + log2f(fmaxf(l_run, 1e-37f))) * 0.6931471805599453f;
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) { tc_fence_after_sync(); tmem_dealloc(tmem_base, TMEM_COLS); }
}

template <int HD, int BN, bool CAUSAL>
static int fwd_set_attr() {
  static bool done = false;
  if (done) return 0;
  constexpr int SMEM = 128 * HD * 2 + 4 * BN * HD * 2 + 128 * BN * 2 + 128;
  (void)cudaGetLastError();
  if (cudaFuncSetAttribute(flash_fwd_kernel<HD, BN, CAUSAL>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess) return 1;
  done = true;
  return 0;
}

template <int HD, int BN, bool CAUSAL>
static int launch_fwd(const FlashArgs& a, cudaStream_t st) {
  CUtensorMap tmQ, tmK, tmV;
  const auto BF = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  if (make_tmap_attn(&tmQ, a.q.ptr, BF, 2, a.hd, a.H, a.Sq, a.B, a.q.sh, a.q.ss, a.q.sb, 64, 128, CU_TENSOR_MAP_SWIZZLE_128B)) return 101;
  if (make_tmap_attn(&tmK, a.k.ptr, BF, 2, a.hd, a.H, a.Skv, a.B, a.k.sh, a.k.ss, a.k.sb, 64, BN, CU_TENSOR_MAP_SWIZZLE_128B)) return 102;
  if (make_tmap_attn(&tmV, a.v.ptr, BF, 2, a.hd, a.H, a.Skv, a.B, a.v.sh, a.v.ss, a.v.sb, 64, BN, CU_TENSOR_MAP_SWIZZLE_128B)) return 103;
  constexpr int SMEM = 128 * HD * 2 + 4 * BN * HD * 2 + 128 * BN * 2 + 128;
  auto kfn = flash_fwd_kernel<HD, BN, CAUSAL>;
  if (fwd_set_attr<HD, BN, CAUSAL>()) return 104;
  FwdParams p;
  p.o = (__nv_bfloat16*)a.o.ptr; p.o_sb = a.o.sb; p.o_ss = a.o.ss; p.o_sh = a.o.sh;
  p.lse = a.lse; p.B = a.B; p.H = a.H; p.Sq = a.Sq; p.Skv = a.Skv;
  p.scale_log2 = a.scale * 1.4426950408889634f;
  p.global_order = ((long long)a.B * a.H * a.Skv * a.hd * 4 <= 300ll * 1024 * 1024) ? 1 : 0;
  p.status = a.status;
  const long long grid = (long long)((a.Sq + 127) / 128) * a.H * a.B;
  cudaError_t e = launch_pdl(kfn, dim3((unsigned)grid), dim3(128), SMEM, st, tmQ, tmK, tmV, p);
  if (e == cudaSuccess) e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}

}  // namespace b200

extern "C" int b200_flash_fwd_init() {
  using namespace b200;
  return fwd_set_attr<64, 128, true>() | fwd_set_attr<64, 128, false>() | fwd_set_attr<128, 64, true>() | fwd_set_attr<128, 64, false>();
}

extern "C" int b200_flash_fwd(const b200::FlashArgs* a, cudaStream_t st) {
  using namespace b200;
  if (a->B <= 0 || a->H <= 0 || a->Sq <= 0 || a->Skv <= 0) return 0;
  if (a->hd == 64) return a->causal ? launch_fwd<64, 128, true>(*a, st) : launch_fwd<64, 128, false>(*a, st);
  if (a->hd == 128) return a->causal ? launch_fwd<128, 64, true>(*a, st) : launch_fwd<128, 64, false>(*a, st);
  return -3;
}
