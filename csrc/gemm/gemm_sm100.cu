// G1: persistent, warp-specialised tcgen05 GEMM for sm_100a.
//
//   C[b] = epilogue( alpha * A[b] * B[b]^T )          A: logical [M,K]   B: logical [N,K]
//
// Either operand may be K-major (stored [rows,K], K contiguous) or MN-major (stored [K,rows],
// rows contiguous); the transposition is expressed in the TMA tensor map and the tensor-core
// matrix descriptor, never as a copy. This is the same contract as the reference's packed CPU
// GEMM, which folds transposes into packing (rust-nn src/blas.rs:104-186, 273-339), and it is the
// one routine behind Linear forward (NT), dX (NN) and dW (TN) (src/tensor.rs:767-781, 1649-1687).
//
// Structure per CTA (320 threads, one CTA per SM, persistent over output tiles):
//   warp 0    : TMA producer  - cp.async.bulk.tensor into a ring of 128B-swizzled stages
//   warp 1    : MMA issuer    - one elected thread issues tcgen05.mma (128 x BN x 16), accumulators
//                               live in TMEM, double-buffered so the epilogue overlaps the next tile
//   warps 2-9 : epilogue      - two warps per TMEM lane quarter, each draining half of the tile's
//                               columns: tcgen05.ld TMEM -> registers (one row per thread), fused bias /
//                               activation / activation gradient / residual, then a transpose through
//                               a per-warp swizzled shared-memory panel so that global stores (and the
//                               residual / saved-activation loads) move whole 128-byte row segments.
//                               fp32 outputs and fp32 atomic accumulation (split-K, gradient
//                               accumulation) are written straight from registers.
// All waits are bounded; on expiry a code lands in the status word and the CTA unwinds.
#include "../common/ptx.cuh"
#include "../common/launch.cuh"
#include "../common/tensormap.h"
#include "gemm_sm100.h"

namespace b200 {

constexpr int BM = 128;
constexpr int EPI_WARPS = 8;
constexpr int GEMM_THREADS = 64 + 32 * EPI_WARPS;   // TMA warp + MMA warp + epilogue warps
constexpr int TILE_K_BYTES = 128;  // one swizzle row
constexpr int UMMA_K_BYTES = 32;
constexpr int EPI_PANEL_BYTES = 32 * 128;   // per-warp staging panel: 32 rows x 128 bytes

template <typename T> struct ElemTraits;
template <> struct ElemTraits<__nv_bfloat16> {
  static constexpr int BK = 64;
  static constexpr uint32_t FMT = FMT_BF16;
  static constexpr bool TF32 = false;
};
template <> struct ElemTraits<float> {
  static constexpr int BK = 32;
  static constexpr uint32_t FMT = FMT_TF32;
  static constexpr bool TF32 = true;
};
// 8-bit operand tags (one byte each). The integer kinds accumulate in int32, fp8 in fp32; the
// epilogue turns either into fp32 and applies per-row (A) and per-column (B) dequantisation scales.
struct s8s8_t { int8_t v; };     // signed x signed      (quantised activations x quantised weights)
struct u8s8_t { uint8_t v; };    // unsigned A x signed B (the reference's igemm contract, src/int8.rs:222-234)
struct e4m3_t { uint8_t v; };    // fp8 e4m3 x e4m3
enum : int { KIND_F16 = 0, KIND_TF32 = 1, KIND_I8 = 2, KIND_F8 = 3 };
template <typename T> struct KindOf { static constexpr int v = ElemTraits<T>::TF32 ? KIND_TF32 : KIND_F16; static constexpr uint32_t AF = ElemTraits<T>::FMT, BF = ElemTraits<T>::FMT, CF = CFMT_F32; };
template <> struct ElemTraits<s8s8_t> { static constexpr int BK = 128; static constexpr uint32_t FMT = FMT_S8; static constexpr bool TF32 = false; };
template <> struct ElemTraits<u8s8_t> { static constexpr int BK = 128; static constexpr uint32_t FMT = FMT_S8; static constexpr bool TF32 = false; };
template <> struct ElemTraits<e4m3_t> { static constexpr int BK = 128; static constexpr uint32_t FMT = 0; static constexpr bool TF32 = false; };
template <> struct KindOf<s8s8_t> { static constexpr int v = KIND_I8; static constexpr uint32_t AF = FMT_S8, BF = FMT_S8, CF = CFMT_S32; };
template <> struct KindOf<u8s8_t> { static constexpr int v = KIND_I8; static constexpr uint32_t AF = FMT_U8, BF = FMT_S8, CF = CFMT_S32; };
template <> struct KindOf<e4m3_t> { static constexpr int v = KIND_F8; static constexpr uint32_t AF = 0, BF = 0, CF = CFMT_F32; };   // 0 = E4M3 in kind::f8f6f4

// hardware tanh (MUFU.TANH): relative error ~2^-11, far below bf16 output precision
__device__ __forceinline__ float tanh_fast(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float act_fwd(float v, int act) {
  switch (act) {
    case ACT_RELU: return v > 0.f ? v : 0.f;
    case ACT_GELU: {
      const float k0 = 0.7978845608028654f, k1 = 0.044715f;
      float u = k0 * (v + k1 * v * v * v);
      return 0.5f * v * (1.f + tanh_fast(u));
    }
    case ACT_SILU: return v / (1.f + __expf(-v));
    case ACT_SIGMOID: return 1.f / (1.f + __expf(-v));
    case ACT_TANH: return tanh_fast(v);
    default: return v;
  }
}
// derivative of the activation, evaluated at the saved value `s`:
// the pre-activation for GELU/SiLU, the output for ReLU/sigmoid/tanh.
__device__ __forceinline__ float act_bwd(float s, int act) {
  switch (act) {
    case ACT_RELU: return s > 0.f ? 1.f : 0.f;
    case ACT_GELU: {
      const float k0 = 0.7978845608028654f, k1 = 0.044715f;
      float u = k0 * (s + k1 * s * s * s);
      float t = tanh_fast(u);
      float du = k0 * (1.f + 3.f * k1 * s * s);
      return 0.5f * (1.f + t) + 0.5f * s * (1.f - t * t) * du;
    }
    case ACT_SILU: {
      float sg = 1.f / (1.f + __expf(-s));
      return sg * (1.f + s * (1.f - sg));
    }
    case ACT_SIGMOID: return s * (1.f - s);
    case ACT_TANH: return 1.f - s * s;
    default: return 1.f;
  }
}

// CG = 2: a pair of CTAs on neighbouring SMs shares one 256 x BN tile; each CTA stages its own 128 rows of A and its own
// half (BN / 2 rows) of B, so a K step moves 32 KB per SM instead of 48 KB for the same FLOPs per SM.
template <typename T, int BN, bool A_MN, bool B_MN, int CG = 1>
struct GemmSmem {
  static constexpr int BK = ElemTraits<T>::BK;
  static constexpr int A_BYTES = BM * TILE_K_BYTES;   // 16 KB
  static constexpr int B_BYTES = (BN / CG) * TILE_K_BYTES;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int EPI_BYTES = EPI_WARPS * EPI_PANEL_BYTES;   // 32 KB
  static constexpr int BAR_BYTES = 256;
  static constexpr int LIMIT = 227 * 1024;
  static constexpr int STAGES_RAW = (LIMIT - EPI_BYTES - BAR_BYTES - 1024) / STAGE_BYTES;
  static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
  static constexpr int TOTAL = STAGES * STAGE_BYTES + EPI_BYTES + BAR_BYTES + 1024;  // +1024: manual alignment
};

// ---------------------------------------------------------------------------- epilogue panel helpers
// A "panel" is the 32 rows x PW columns (bf16) a warp holds with one row per thread. It is moved
// through a per-warp shared-memory buffer (rows of PW*2 bytes, 16-byte chunks XOR-swizzled so both
// the row-owner accesses and the coalesced accesses are bank-conflict free) so that every global
// load / store instruction of the warp touches RPI complete row segments of PW*2 bytes.
template <int PW>
struct Panel {
  static constexpr int CPR = PW / 8;          // 16-byte chunks per row
  static constexpr int RPI = 32 / CPR;        // rows per warp-wide instruction
  static constexpr int NI = 32 / RPI;         // instructions per panel
  static constexpr int ROW_BYTES = PW * 2;
  __device__ static __forceinline__ uint32_t off(int row, int chunk) {
    const int sw = (PW == 64) ? (row & 7) : ((row >> 1) & 3);
    return row * ROW_BYTES + ((chunk ^ sw) << 4);
  }
};

// registers (row owner: this lane = row `lane`, PW fp32 values) -> bf16 -> global, coalesced
template <int PW>
__device__ __forceinline__ void panel_store(uint8_t* sbuf, int lane, const float (&f)[PW], __nv_bfloat16* gpanel,
                                            long long ld, int rows_valid, int chunks_valid) {
  using P = Panel<PW>;
  __syncwarp();
#pragma unroll
  for (int c = 0; c < P::CPR; ++c) {
    uint4 o = make_uint4(pack_bf16x2(f[8 * c], f[8 * c + 1]), pack_bf16x2(f[8 * c + 2], f[8 * c + 3]),
                         pack_bf16x2(f[8 * c + 4], f[8 * c + 5]), pack_bf16x2(f[8 * c + 6], f[8 * c + 7]));
    *reinterpret_cast<uint4*>(sbuf + P::off(lane, c)) = o;
  }
  __syncwarp();
  const int c = lane % P::CPR, r0 = lane / P::CPR;
#pragma unroll
  for (int i = 0; i < P::NI; ++i) {
    const int row = i * P::RPI + r0;
    const uint4 v = *reinterpret_cast<const uint4*>(sbuf + P::off(row, c));
    if (row < rows_valid && c < chunks_valid) *reinterpret_cast<uint4*>(gpanel + (long long)row * ld + c * 8) = v;
  }
}

// Tensor maps of the bf16 outputs (C and the optional pre-activation copy), box {64 columns, 32 rows}: with them a warp
// hands its 32 x 64 panel to the TMA engine as ONE store instead of reading it back from shared memory and issuing
// 8 predicated 16-byte stores per thread.
struct OutMaps {
  CUtensorMap c, aux;
  int use;              // 0: plain stores (fp32 / int32 outputs, unaligned C, narrow tiles)
};

// GEMM -> reduce-scatter: one map per rank over ITS slot buffer [2 * world][rows_per_rank][N] (peer-mapped), so that a
// panel crosses NVLink as one bulk store instead of 256 16-byte stores (no load, and nothing multicast, goes that way)
struct PeerMaps {
  CUtensorMap m[TP_MAX_WORLD];
  int use;
};

// registers (row owner) -> bf16 panel in the 128-byte-swizzle layout -> one TMA store; rows and columns past the edge of
// the tensor are clipped by the copy engine. The panel buffer is reused, so the previous store's read of it is awaited first.
__device__ __forceinline__ void panel_store_tma(uint8_t* sbuf, int lane, const float (&f)[64], const CUtensorMap* tm, int col0, int row0, int b) {
  if (lane == 0) tma_store_wait_read0();
  __syncwarp();
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    uint4 o = make_uint4(pack_bf16x2(f[8 * c], f[8 * c + 1]), pack_bf16x2(f[8 * c + 2], f[8 * c + 3]),
                         pack_bf16x2(f[8 * c + 4], f[8 * c + 5]), pack_bf16x2(f[8 * c + 6], f[8 * c + 7]));
    *reinterpret_cast<uint4*>(sbuf + sw128_offset(lane, c)) = o;
  }
  fence_proxy_async_smem();
  __syncwarp();
  if (lane == 0) { tma_store_3d(tm, sbuf, col0, row0, b); tma_store_commit(); }
}

// global (bf16, coalesced) -> row-owner registers: out[c] = 8 bf16 of this lane's row, chunk c
template <int PW>
__device__ __forceinline__ void panel_load(uint8_t* sbuf, int lane, const __nv_bfloat16* gpanel, long long ld,
                                           int rows_valid, int chunks_valid, uint4 (&out)[PW / 8]) {
  using P = Panel<PW>;
  __syncwarp();
  const int c = lane % P::CPR, r0 = lane / P::CPR;
#pragma unroll
  for (int i = 0; i < P::NI; ++i) {
    const int row = i * P::RPI + r0;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (row < rows_valid && c < chunks_valid) v = *reinterpret_cast<const uint4*>(gpanel + (long long)row * ld + c * 8);
    *reinterpret_cast<uint4*>(sbuf + P::off(row, c)) = v;
  }
  __syncwarp();
#pragma unroll
  for (int cc = 0; cc < P::CPR; ++cc) out[cc] = *reinterpret_cast<const uint4*>(sbuf + P::off(lane, cc));
}

// ---------------------------------------------------------------------------- peer-memory helpers (TP variants)
__device__ __forceinline__ void st_release_sys_u32(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu_u32(uint32_t* p, uint32_t v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_gpu_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }
// bounded spin until *p >= want (wrap-safe); false (and a status code) on expiry
template <bool SYS>
__device__ __forceinline__ bool wait_flag(const uint32_t* p, uint32_t want, long long budget, uint32_t* status, uint32_t code) {
  const long long t0 = clock64();
  while ((int32_t)((SYS ? ld_acquire_sys_u32(p) : ld_acquire_gpu_u32(p)) - want) < 0) {
    if (clock64() - t0 > budget) { if (status) atomicCAS(status, 0u, code); return false; }
    __nanosleep(128);
  }
  return true;
}
// one thread: tell every peer `which` (0: shard ready, 1: done) and, if `wait`, wait for all of them
__device__ __forceinline__ bool peer_handshake(const TpParams& tp, uint32_t epoch, int which, bool wait, uint32_t* status) {
  __threadfence_system();
  for (int r = 0; r < tp.world; ++r) st_release_sys_u32(tp.flags[r] + which * TP_MAX_WORLD + tp.rank, epoch);
  bool ok = true;
  if (wait)
    for (int r = 0; r < tp.world && ok; ++r)
      ok = wait_flag<true>(tp.flags[tp.rank] + which * TP_MAX_WORLD + r, epoch, tp.wait_cycles, status, ST_TIMEOUT_PEER_FLAG);
  return ok;
}

// KEEP_PERMIT: the kernel will allocate tensor memory again after this body (a fused kernel that runs two products):
// the allocation permit is then not given up here (no allocation is legal after `relinquish_alloc_permit`).
template <typename T, int BN, bool A_MN, bool B_MN, int TP, int CG = 1, bool KEEP_PERMIT = false>
__device__ __forceinline__ void gemm_body(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p, const TpParams* tpp,
                                          const OutMaps* om = nullptr, const PeerMaps* pm = nullptr) {
  using S = GemmSmem<T, BN, A_MN, B_MN, CG>;
  static_assert(CG == 1 || (CG == 2 && TP == TP_NONE && BN == 256), "CTA pairs: plain GEMM with 256-wide tiles only");
  constexpr int BNL = BN / CG;                          // rows of B this CTA stages
  const uint32_t crank = CG == 2 ? cluster_ctarank() : 0u;
  constexpr int BK = S::BK;
  constexpr int STAGES = S::STAGES;
  constexpr int ATOM = TILE_K_BYTES / sizeof(T);        // elements per 128-byte row
  constexpr int UMMA_K = UMMA_K_BYTES / sizeof(T);
  constexpr int K_STEPS = BK / UMMA_K;                  // 4
  constexpr uint32_t TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* epi_smem = smem + STAGES * S::STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(epi_smem + S::EPI_BYTES);
  uint64_t* full_bar = bars;                 // [STAGES]
  uint64_t* empty_bar = bars + STAGES;       // [STAGES]
  uint64_t* acc_full = bars + 2 * STAGES;    // [2]
  uint64_t* acc_empty = bars + 2 * STAGES + 2;  // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  pdl_trigger();

  const int m_blocks = (p.M + BM * CG - 1) / (BM * CG);      // row blocks of a tile: 128 rows, 256 for a CTA pair
  const int n_blocks = (p.N + BN - 1) / BN;
  const int num_kb = (p.K + BK - 1) / BK;
  const int kb_per_split = (num_kb + p.splits - 1) / p.splits;
  // ragged groups: is the row tile of batch `bb` in use, and where does its K loop end
  auto tile_skipped = [&](int bb, int mb_) -> bool { return p.m_valid != nullptr && mb_ * (BM * CG) >= *reinterpret_cast<volatile const int*>(p.m_valid + bb); };
  auto kb_end = [&](int bb) -> int {
    if (p.k_valid == nullptr) return num_kb;
    const int kv = min(p.K, ((*reinterpret_cast<volatile const int*>(p.k_valid + bb) + 127) / 128) * 128);
    return (kv + BK - 1) / BK;
  };
  const long long tiles_per_batch = (long long)m_blocks * n_blocks * p.splits;
  const long long total_tiles = tiles_per_batch * p.batch;
  // TP_AG_GEMM reserves the first `copy_ctas` CTAs for pulling remote shards; the rest run the GEMM
  const int n_copy = (TP == TP_AG_GEMM) ? tpp->copy_ctas : 0;
  const int cta = CG == 2 ? (int)(blockIdx.x >> 1) : (int)blockIdx.x - n_copy;          // CTA pairs walk the tiles together
  const int n_ctas = CG == 2 ? (int)(gridDim.x >> 1) : (int)gridDim.x - n_copy;
  // Row-block order of a tensor-parallel call. all-gather -> GEMM starts with the local rows (the others are still
  // arriving). GEMM -> reduce-scatter starts with the rows of the NEXT rank: every rank then stores into a different
  // owner at any moment; with one common order all ranks would write to owner 0 first, then to owner 1, ..., and the
  // NVLink ingress of one GPU at a time would carry the traffic of all of them.
  const int tp_shift = (TP == TP_AG_GEMM) ? tpp->rank * tpp->blocks_per_rank
                     : (TP == TP_GEMM_RS) ? ((tpp->rank + 1) % tpp->world) * tpp->blocks_per_rank : 0;
  // q-th row block a CTA works on -> row block of the matrix. all-gather -> GEMM: the local rows, then the peers' rows
  // interleaved (block g of rank+1, block g of rank+2, ..., block g+1 of rank+1, ...): that is the order in which the
  // gather CTAs of the peers deliver them, each of them sending its blocks to all its peers at the same pace.
  auto row_block = [&](int q) -> int {
    if constexpr (TP == TP_AG_GEMM) {
      const int bpr = tpp->blocks_per_rank, w = tpp->world;
      if (q < bpr || w <= 1) return (q + tp_shift) % m_blocks;
      const int qq = q - bpr;
      return ((tpp->rank + 1 + qq % (w - 1)) % w) * bpr + qq / (w - 1);
    } else {
      return (q + tp_shift) % m_blocks;
    }
  };
  // The handshake epoch of a tensor-parallel call lives in device memory (one word per context) and is advanced by the
  // call's last CTA, so a CUDA-graph replay of the launch sees a fresh epoch every time.
  const uint32_t tp_epoch = (TP != TP_NONE) ? *reinterpret_cast<volatile const uint32_t*>(tpp->epoch_ptr) + 1u : 0u;

  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; ++i) { mbar_init(&full_bar[i], 1); mbar_init(&empty_bar[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&acc_full[i], 1); mbar_init(&acc_empty[i], EPI_WARPS * CG); }   // pair: both CTAs' epilogue warps arrive at the even CTA
    fence_barrier_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if constexpr (CG == 2) cluster_sync_all();            // the partner's barriers exist before anything is counted on them
  if (warp == 1) {
    if constexpr (CG == 2) { tmem_alloc_pair(tmem_slot, TMEM_COLS); tmem_relinquish_pair(); }
    else { tmem_alloc(tmem_slot, TMEM_COLS); if constexpr (!KEEP_PERMIT) tmem_relinquish(); }
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();                      // everything above overlapped the previous kernel; global memory is touched from here on

  if (TP == TP_AG_GEMM && cta < 0) {
    // ------------------------------------------------------------------ gather CTAs (all-gather half of TP_AG_GEMM)
    // Push model: this rank's rows (already in its staging buffer by stream order) are written into every
    // peer's staging buffer - posted NVLink stores, 8 x 16 bytes in flight per thread - followed by a
    // release of the row block's flag AT THE PEER.
    const TpParams& tp = *tpp;
    uint32_t mover_phase = 0;
    const long long row_bytes = (long long)p.K * 2;                      // bf16 rows, K % 8 == 0
    const long long blk_vec = (long long)BM * row_bytes / 16;            // 16-byte vectors per row block
    constexpr int UNROLL = 8;
    // a system-scope fence drains every outstanding NVLink store, so it is paid once per GROUP row blocks; the group
    // shrinks when there are fewer row blocks than 4 per gather CTA, so that every gather CTA has work
    const int GROUP = max(1, min(4, tp.blocks_per_rank / max(n_copy, 1)));
    const int n_groups = (tp.blocks_per_rank + GROUP - 1) / GROUP;
    const bool bulk = pm != nullptr && (pm->use & 2) != 0;
    if (bulk) {
      // Bulk movers: lane 0 of each of the first MOVERS warps owns one 32 KB buffer of this CTA's (otherwise idle) stage
      // memory and runs load (local staging -> shared) / store (shared -> every peer's staging) chains through the copy
      // engine: no registers in the data path and ~200 KB in flight per CTA.
      constexpr int MOVERS = STAGES < 6 ? STAGES : 6, CH = 32 * 1024;       // one load barrier and (at least) 32 KB of stage memory each
      for (int jg = (int)blockIdx.x; jg < n_groups; jg += n_copy) {
        const int j0 = jg * GROUP;
        const int nblk = min(GROUP, tp.blocks_per_rank - j0);
        const int mbg = tp.rank * tp.blocks_per_rank + j0;
        const long long boff = (long long)mbg * BM * row_bytes;
        const long long grp_bytes = (long long)nblk * BM * row_bytes;        // multiple of 16
        if (lane == 0 && warp < MOVERS) {
          uint8_t* buf = smem + warp * CH;
          uint64_t* bar = &full_bar[warp];
          const uint8_t* src = reinterpret_cast<const uint8_t*>(tp.stage_peer[tp.rank]) + boff;
          bool okm = true;
          for (long long off = (long long)warp * CH; off < grp_bytes && okm; off += (long long)MOVERS * CH) {
            const uint32_t n = (uint32_t)min((long long)CH, grp_bytes - off);
            mbar_expect_tx(bar, n);
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                         ::"r"(smem_u32(buf)), "l"(reinterpret_cast<uint64_t>(src + off)), "r"(n), "r"(smem_u32(bar)) : "memory");
            okm = mbar_wait(bar, mover_phase, p.status, ST_TIMEOUT_TMA_FULL);
            mover_phase ^= 1;
            if (!okm) break;
            for (int rr = 1; rr < tp.world; ++rr) {
              const int peer = (tp.rank + rr) % tp.world;                    // stagger the peers
              uint8_t* dst = reinterpret_cast<uint8_t*>(tp.stage_peer[peer]) + boff + off;
              asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                           ::"l"(reinterpret_cast<uint64_t>(dst)), "r"(smem_u32(buf)), "r"(n) : "memory");
            }
            tma_store_commit();
            tma_store_wait_read0();                                          // the buffer may be refilled
          }
          tma_store_wait0();                                                 // this mover's stores have landed
          fence_proxy_async_all();
        }
        __threadfence_system();
        __syncthreads();
        if (threadIdx.x == 0)
          for (int rr = 1; rr < tp.world; ++rr)
            for (int q = 0; q < nblk; ++q) st_release_sys_u32(tp.ready_peer[(tp.rank + rr) % tp.world] + mbg + q, tp_epoch);
        __syncthreads();
      }
    } else
    for (int jg = (int)blockIdx.x; jg < n_groups; jg += n_copy) {
      const int j0 = jg * GROUP;
      const int nblk = min(GROUP, tp.blocks_per_rank - j0);
      const int mbg = tp.rank * tp.blocks_per_rank + j0;                 // first global row block of the group
      const long long boff = (long long)mbg * BM * row_bytes;
      const long long grp_vec = blk_vec * nblk;
      const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(tp.stage_peer[tp.rank]) + boff);
      for (long long v0 = threadIdx.x; v0 < grp_vec; v0 += (long long)GEMM_THREADS * UNROLL) {
        uint4 x[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
          const long long v = v0 + (long long)u * GEMM_THREADS;
          if (v < grp_vec) x[u] = src[v];
        }
        for (int rr = 1; rr < tp.world; ++rr) {
          const int peer = (tp.rank + rr) % tp.world;                    // stagger the peers
          uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(tp.stage_peer[peer]) + boff);
#pragma unroll
          for (int u = 0; u < UNROLL; ++u) {
            const long long v = v0 + (long long)u * GEMM_THREADS;
            if (v < grp_vec) dst[v] = x[u];
          }
        }
      }
      __threadfence_system();
      __syncthreads();
      if (threadIdx.x == 0)
        for (int rr = 1; rr < tp.world; ++rr)
          for (int q = 0; q < nblk; ++q) st_release_sys_u32(tp.ready_peer[(tp.rank + rr) % tp.world] + mbg + q, tp_epoch);
      __syncthreads();
    }
  } else if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0; bool ok = true;
      for (long long t = cta; t < total_tiles && ok; t += n_ctas) {
        const int b = (int)(t / tiles_per_batch);
        long long r = t % tiles_per_batch;
        const int split = (int)(r / ((long long)m_blocks * n_blocks));
        r %= (long long)m_blocks * n_blocks;
        const int mb = row_block((int)(r / n_blocks)), nb = (int)(r % n_blocks);
        if (tile_skipped(b, mb)) continue;
        const int kb0 = split * kb_per_split;
        const int kb1 = min(kb0 + kb_per_split, kb_end(b));
        if constexpr (TP == TP_AG_GEMM) {
          // rows of another rank: wait until the gather CTAs have landed this row block
          if (mb / tpp->blocks_per_rank != tpp->rank) {
            if (!wait_flag<true>(tpp->ready_peer[tpp->rank] + mb, tp_epoch, tpp->wait_cycles, p.status, ST_TIMEOUT_PEER_FLAG)) { ok = false; break; }
            fence_proxy_async_all();
          }
        }
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, p.status, ST_TIMEOUT_TMA_EMPTY)) { ok = false; break; }
          uint8_t* sa = smem + stage * S::STAGE_BYTES;
          uint8_t* sb = sa + S::A_BYTES;
          if constexpr (CG == 2) {
            // both CTAs load their own halves; the bytes of both are counted on the even CTA's barrier, which its MMA thread waits on
            const int arow = (mb * 2 + (int)crank) * BM, brow = nb * BN + (int)crank * BNL;
            const uint32_t bar = cluster_map(smem_u32(&full_bar[stage]), 0);
            if (crank == 0) mbar_expect_tx(&full_bar[stage], 2 * S::STAGE_BYTES);
            if (!A_MN) {
              tma_load_3d_pair(sa, &tmA, bar, kb * BK, arow, b);
            } else {
#pragma unroll
              for (int a = 0; a < BM / ATOM; ++a)
                tma_load_3d_pair(sa + a * (BK * TILE_K_BYTES), &tmA, bar, arow + a * ATOM, kb * BK, b);
            }
            if (!B_MN) {
              tma_load_3d_pair(sb, &tmB, bar, kb * BK, brow, b);
            } else {
#pragma unroll
              for (int a = 0; a < BNL / ATOM; ++a)
                tma_load_3d_pair(sb + a * (BK * TILE_K_BYTES), &tmB, bar, brow + a * ATOM, kb * BK, b);
            }
            if (++stage == STAGES) { stage = 0; phase ^= 1; }
            continue;
          }
          mbar_expect_tx(&full_bar[stage], S::STAGE_BYTES);
          if (!A_MN) {
            tma_load_3d(sa, &tmA, &full_bar[stage], kb * BK, mb * BM, b);
          } else {
#pragma unroll
            for (int a = 0; a < BM / ATOM; ++a)
              tma_load_3d(sa + a * (BK * TILE_K_BYTES), &tmA, &full_bar[stage], mb * BM + a * ATOM, kb * BK, b);
          }
          if (!B_MN) {
            tma_load_3d(sb, &tmB, &full_bar[stage], kb * BK, nb * BN, b);
          } else {
#pragma unroll
            for (int a = 0; a < BN / ATOM; ++a)
              tma_load_3d(sb + a * (BK * TILE_K_BYTES), &tmB, &full_bar[stage], nb * BN + a * ATOM, kb * BK, b);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && crank == 0) {                       // of a CTA pair only the even CTA issues
      constexpr uint32_t idesc = make_idesc(BM * CG, BN, KindOf<T>::CF, KindOf<T>::AF, KindOf<T>::BF,
                                            A_MN ? 1u : 0u, B_MN ? 1u : 0u);
      // K-major: 8-row groups 1024 B apart.  MN-major: 8-k-row groups 1024 B apart, 128B-row atoms
      // BK*128 B apart.
      constexpr uint32_t A_LBO = A_MN ? BK * TILE_K_BYTES : 0, A_SBO = 1024;
      constexpr uint32_t B_LBO = B_MN ? BK * TILE_K_BYTES : 0, B_SBO = 1024;
      constexpr uint32_t A_KADV = A_MN ? UMMA_K * TILE_K_BYTES : UMMA_K_BYTES;
      constexpr uint32_t B_KADV = B_MN ? UMMA_K * TILE_K_BYTES : UMMA_K_BYTES;
      int stage = 0; uint32_t phase = 0; bool ok = true;
      int it = 0;                                   // tiles this CTA really computes (skipped ones use no accumulator)
      for (long long t = cta; t < total_tiles && ok; t += n_ctas) {
        const int b = (int)(t / tiles_per_batch);
        long long r = t % tiles_per_batch;
        const int split = (int)(r / ((long long)m_blocks * n_blocks));
        r %= (long long)m_blocks * n_blocks;
        if (tile_skipped(b, row_block((int)(r / n_blocks)))) continue;
        const int kb0 = split * kb_per_split;
        const int kb1 = min(kb0 + kb_per_split, kb_end(b));
        const int as = it & 1;
        const uint32_t aphase = (it >> 1) & 1;
        if (!mbar_wait(&acc_empty[as], aphase ^ 1, p.status, ST_TIMEOUT_ACC_EMPTY)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + as * BN;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, p.status, ST_TIMEOUT_TMA_FULL)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem + stage * S::STAGE_BYTES);
          const uint32_t sb = sa + S::A_BYTES;
#pragma unroll
          for (int k = 0; k < K_STEPS; ++k) {
            uint64_t da = make_sdesc_sw128(sa + k * A_KADV, A_LBO, A_SBO);
            uint64_t db = make_sdesc_sw128(sb + k * B_KADV, B_LBO, B_SBO);
            const uint32_t accum = (kb > kb0 || k > 0) ? 1u : 0u;
            if constexpr (CG == 2) umma_f16_pair(d_tmem, da, db, idesc, accum);
            else if constexpr (KindOf<T>::v == KIND_TF32) umma_tf32(d_tmem, da, db, idesc, accum);
            else if constexpr (KindOf<T>::v == KIND_I8) umma_i8(d_tmem, da, db, idesc, accum);
            else if constexpr (KindOf<T>::v == KIND_F8) umma_f8(d_tmem, da, db, idesc, accum);
            else umma_f16(d_tmem, da, db, idesc, accum);
          }
          if constexpr (CG == 2) {          // the stage is free in BOTH CTAs once these MMAs have read it
            tc_commit_pair(cluster_map(smem_u32(&empty_bar[stage]), 0));
            tc_commit_pair(cluster_map(smem_u32(&empty_bar[stage]), 1));
          } else {
            tc_commit(&empty_bar[stage]);   // stage reusable once these MMAs have read it
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) {
          if constexpr (CG == 2) {
            tc_commit_pair(cluster_map(smem_u32(&acc_full[as]), 0));
            tc_commit_pair(cluster_map(smem_u32(&acc_full[as]), 1));
          } else {
            tc_commit(&acc_full[as]);
          }
        }
        ++it;
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..9)
    const int ew = warp - 2;
    const int q = warp & 3;                      // TMEM lane quarter this warp may read
    const int chalf = ew >> 2;                   // which half of the tile's columns this warp drains
    constexpr int CPW = BN / 2;                  // columns per warp (32, 64 or 128)
    constexpr int PW = CPW >= 64 ? 64 : 32;      // panel width
    constexpr int NPANEL = CPW / PW;
    uint8_t* sbuf = epi_smem + ew * EPI_PANEL_BYTES;
    const float alpha = p.alpha_ptr ? p.alpha * __ldg(p.alpha_ptr) : p.alpha;
    const bool staged = (p.out_mode == OUT_BF16) && p.vec_ok;       // coalesced bf16 path
    const bool tma_out = staged && PW == 64 && TP != TP_GEMM_RS && om != nullptr && om->use;   // ... through the TMA engine
    const bool rs_tma = staged && PW == 64 && TP == TP_GEMM_RS && pm != nullptr && pm->use;    // partial tiles to their owners, ditto
    bool ok = true;
    int it = 0;
    for (long long t = cta; t < total_tiles && ok; t += n_ctas) {
      const int b = (int)(t / tiles_per_batch);
      long long r = t % tiles_per_batch;
      const int split = (int)(r / ((long long)m_blocks * n_blocks));
      r %= (long long)m_blocks * n_blocks;
      const int mb = row_block((int)(r / n_blocks)), nb = (int)(r % n_blocks);
      if (tile_skipped(b, mb)) continue;
      const int kb0 = split * kb_per_split;
      const bool has_k = kb0 < min(kb0 + kb_per_split, kb_end(b));
      const int as = it & 1;
      const uint32_t aphase = (it >> 1) & 1;
      if (!mbar_wait(&acc_full[as], aphase, p.status, ST_TIMEOUT_ACC_FULL)) { ok = false; break; }
      tc_fence_after_sync();
      const int row0 = (mb * CG + (int)crank) * BM + q * 32;          // first row of this warp's panel
      const int row = row0 + lane;
      const bool row_ok = row < p.M;
      const int rows_valid = min(32, p.M - row0);  // may be <= 0
      const long long cbase = (long long)b * p.strideC + (long long)row0 * p.ldc;   // element offset of (row0, 0)
      const long long rbase = (long long)b * p.strideR + (long long)row0 * p.ldr;
      const bool first_split = (split == 0);
      const uint32_t tbase = tmem_base + (uint32_t(q * 32) << 16) + as * BN + chalf * CPW;
#pragma unroll 1
      for (int pn = 0; pn < NPANEL; ++pn) {
        const int col0 = nb * BN + chalf * CPW + pn * PW;
        uint32_t v[PW];
#pragma unroll
        for (int c = 0; c < PW / 32; ++c) tmem_ld_x32(tbase + pn * PW + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&v[c * 32]));
        tmem_ld_wait();
        if (rows_valid <= 0 || col0 >= p.N) continue;
        const int cols_valid = min(PW, p.N - col0);
        const int chunks_valid = cols_valid / 8;       // staged path has N % 8 == 0
        const bool full = cols_valid == PW;
        if constexpr (KindOf<T>::v == KIND_I8) {
          if (p.out_mode == OUT_I32) {       // raw integer accumulators (igemm contract)
            if (row_ok) {
              int* cp = reinterpret_cast<int*>(p.C) + cbase + (long long)lane * p.ldc + col0;
              if (full && p.vec_ok) {
#pragma unroll
                for (int j = 0; j < PW; j += 4)
                  *reinterpret_cast<int4*>(cp + j) = has_k ? make_int4((int)v[j], (int)v[j + 1], (int)v[j + 2], (int)v[j + 3]) : make_int4(0, 0, 0, 0);
              } else {
#pragma unroll
                for (int j = 0; j < PW; ++j) if (j < cols_valid) cp[j] = has_k ? (int)v[j] : 0;
              }
            }
            continue;
          }
        }
        float f[PW];
        if constexpr (KindOf<T>::v == KIND_I8) {
#pragma unroll
          for (int j = 0; j < PW; ++j) f[j] = has_k ? (float)(int)v[j] * alpha : 0.f;
        } else {
#pragma unroll
          for (int j = 0; j < PW; ++j) f[j] = has_k ? __uint_as_float(v[j]) * alpha : 0.f;
        }
        if (p.row_scale || p.col_scale) {
          // dequantise: per-row scale of A (one per thread's row) and per-column scale of B
          const float rs = (p.row_scale && row_ok) ? __ldg(p.row_scale + (long long)b * p.M + row) : 1.f;
          if (p.col_scale) {
            const float* cs = p.col_scale + col0;
#pragma unroll
            for (int j = 0; j < PW; ++j) f[j] *= rs * ((j < cols_valid) ? __ldg(cs + j) : 0.f);
          } else {
#pragma unroll
            for (int j = 0; j < PW; ++j) f[j] *= rs;
          }
        }
        if (p.bias && first_split) {
          if (p.bias_f32 && full && p.bias_vec_ok) {
            const float4* bp = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.bias) + b * p.strideBias + col0);
#pragma unroll
            for (int j = 0; j < PW / 4; ++j) {
              const float4 bb = __ldg(bp + j);
              f[4 * j] += bb.x; f[4 * j + 1] += bb.y; f[4 * j + 2] += bb.z; f[4 * j + 3] += bb.w;
            }
          } else if (p.bias_f32) {
            const float* bp = reinterpret_cast<const float*>(p.bias) + b * p.strideBias + col0;
#pragma unroll
            for (int j = 0; j < PW; ++j) if (j < cols_valid) f[j] += __ldg(bp + j);
          } else {
            const __nv_bfloat16* bp = reinterpret_cast<const __nv_bfloat16*>(p.bias) + b * p.strideBias + col0;
#pragma unroll
            for (int j = 0; j < PW; ++j) if (j < cols_valid) f[j] += __bfloat162float(bp[j]);
          }
        }
        if (p.aux_out) {          // bf16 copy of the pre-activation (dense layout of C)
          __nv_bfloat16* ap = reinterpret_cast<__nv_bfloat16*>(p.aux_out) + cbase + col0;
          if constexpr (PW == 64) {
            if (tma_out) panel_store_tma(sbuf, lane, f, &om->aux, col0, row0, b);
          }
          if (tma_out) {}
          else if (staged) panel_store<PW>(sbuf, lane, f, ap, p.ldc, rows_valid, chunks_valid);
          else if (row_ok) {
#pragma unroll
            for (int j = 0; j < PW; ++j) if (j < cols_valid) ap[(long long)lane * p.ldc + j] = __float2bfloat16(f[j]);
          }
        }
        // the activation switch sits OUTSIDE the element loops: one straight-line loop per case keeps
        // the unrolled epilogue small enough for the instruction cache
        switch (p.act) {
#define B200_ACT_CASE(A) case A: { _Pragma("unroll") for (int j = 0; j < PW; ++j) f[j] = act_fwd(f[j], A); } break;
          B200_ACT_CASE(ACT_RELU) B200_ACT_CASE(ACT_GELU) B200_ACT_CASE(ACT_SILU) B200_ACT_CASE(ACT_SIGMOID) B200_ACT_CASE(ACT_TANH)
#undef B200_ACT_CASE
          default: break;
        }
        if (p.aux_in) {           // multiply by act'(saved)
          const __nv_bfloat16* ap = reinterpret_cast<const __nv_bfloat16*>(p.aux_in) + cbase + col0;
          if (staged) {
            uint4 u[PW / 8];
            if (tma_out) { if (lane == 0) tma_store_wait_read0(); __syncwarp(); }
            panel_load<PW>(sbuf, lane, ap, p.ldc, rows_valid, chunks_valid, u);
            switch (p.dact) {
#define B200_DACT_CASE(A) case A: { _Pragma("unroll") for (int j = 0; j < PW / 8; ++j) { \
                const float2 a0 = unpack_bf16x2(u[j].x), a1 = unpack_bf16x2(u[j].y), a2 = unpack_bf16x2(u[j].z), a3 = unpack_bf16x2(u[j].w); \
                f[8 * j] *= act_bwd(a0.x, A); f[8 * j + 1] *= act_bwd(a0.y, A); f[8 * j + 2] *= act_bwd(a1.x, A); f[8 * j + 3] *= act_bwd(a1.y, A); \
                f[8 * j + 4] *= act_bwd(a2.x, A); f[8 * j + 5] *= act_bwd(a2.y, A); f[8 * j + 6] *= act_bwd(a3.x, A); f[8 * j + 7] *= act_bwd(a3.y, A); } } break;
              B200_DACT_CASE(ACT_RELU) B200_DACT_CASE(ACT_GELU) B200_DACT_CASE(ACT_SILU) B200_DACT_CASE(ACT_SIGMOID) B200_DACT_CASE(ACT_TANH)
#undef B200_DACT_CASE
              default: break;
            }
          } else if (row_ok) {
#pragma unroll
            for (int j = 0; j < PW; ++j) if (j < cols_valid) f[j] *= act_bwd(__bfloat162float(ap[(long long)lane * p.ldc + j]), p.dact);
          }
        }
        if (TP != TP_GEMM_RS && p.residual && first_split) {       // TP_GEMM_RS adds the residual after the reduction
          const __nv_bfloat16* rp = reinterpret_cast<const __nv_bfloat16*>(p.residual) + rbase + col0;
          if (staged && p.res_vec_ok) {
            uint4 u[PW / 8];
            if (tma_out) { if (lane == 0) tma_store_wait_read0(); __syncwarp(); }
            panel_load<PW>(sbuf, lane, rp, p.ldr, rows_valid, chunks_valid, u);
#pragma unroll
            for (int j = 0; j < PW / 8; ++j) {
              const float2 a0 = unpack_bf16x2(u[j].x), a1 = unpack_bf16x2(u[j].y), a2 = unpack_bf16x2(u[j].z), a3 = unpack_bf16x2(u[j].w);
              f[8 * j] += a0.x; f[8 * j + 1] += a0.y; f[8 * j + 2] += a1.x; f[8 * j + 3] += a1.y;
              f[8 * j + 4] += a2.x; f[8 * j + 5] += a2.y; f[8 * j + 6] += a3.x; f[8 * j + 7] += a3.y;
            }
          } else if (row_ok) {
#pragma unroll
            for (int j = 0; j < PW; ++j) if (j < cols_valid) f[j] += __bfloat162float(rp[(long long)lane * p.ldr + j]);
          }
        }
        if (p.out_mode == OUT_BF16) {
          __nv_bfloat16* cp = reinterpret_cast<__nv_bfloat16*>(p.C) + cbase + col0;
          if constexpr (TP == TP_GEMM_RS) {
            // this row block belongs to rank `owner`: store into MY slot of ITS buffer (peer memory, plain stores)
            const TpParams& tp = *tpp;
            const int owner = mb / tp.blocks_per_rank;
            const long long rows_per_rank = (long long)tp.blocks_per_rank * BM;
            const long long slot = ((long long)(tp_epoch & 1u) * tp.world + tp.rank) * rows_per_rank;
            cp = reinterpret_cast<__nv_bfloat16*>(tp.slots_peer[owner]) + (slot + (row0 - owner * rows_per_rank)) * p.ldc + col0;
          }
          if constexpr (PW == 64) {
            if (tma_out) panel_store_tma(sbuf, lane, f, &om->c, col0, row0, b);
            if constexpr (TP == TP_GEMM_RS) {
              if (rs_tma) {
                const TpParams& tp = *tpp;
                const int owner = mb / tp.blocks_per_rank;
                panel_store_tma(sbuf, lane, f, &pm->m[owner], col0, row0 - owner * tp.blocks_per_rank * BM, (int)(tp_epoch & 1u) * tp.world + tp.rank);
              }
            }
          }
          if (tma_out || rs_tma) {}
          else if (staged) panel_store<PW>(sbuf, lane, f, cp, p.ldc, rows_valid, chunks_valid);
          else if (row_ok) {
#pragma unroll
            for (int j = 0; j < PW; ++j) if (j < cols_valid) cp[(long long)lane * p.ldc + j] = __float2bfloat16(f[j]);
          }
        } else if (row_ok) {
          float* cp = reinterpret_cast<float*>(p.C) + cbase + (long long)lane * p.ldc + col0;
          const bool vec = full && p.vec_ok;
          if (p.out_mode == OUT_F32) {
            if (vec) {
#pragma unroll
              for (int j = 0; j < PW; j += 4) *reinterpret_cast<float4*>(cp + j) = make_float4(f[j], f[j + 1], f[j + 2], f[j + 3]);
            } else {
#pragma unroll
              for (int j = 0; j < PW; ++j) if (j < cols_valid) cp[j] = f[j];
            }
          } else {  // OUT_F32_ATOMIC
            if (vec) {
#pragma unroll
              for (int j = 0; j < PW; j += 4) atomicAdd(reinterpret_cast<float4*>(cp + j), make_float4(f[j], f[j + 1], f[j + 2], f[j + 3]));
            } else {
#pragma unroll
              for (int j = 0; j < PW; ++j) if (j < cols_valid) atomicAdd(cp + j, f[j]);
            }
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        if constexpr (CG == 2) mbar_arrive_cluster(cluster_map(smem_u32(&acc_empty[as]), 0));
        else mbar_arrive(&acc_empty[as]);
      }
      ++it;
    }
    if ((tma_out || rs_tma) && lane == 0) {               // this warp's last stores have left shared memory and landed
      tma_store_wait0();
      if (rs_tma) { fence_proxy_async_all(); __threadfence_system(); }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if constexpr (CG == 2) cluster_sync_all();            // neither CTA leaves (or frees TMEM) while its partner may still use it
  if (warp == 1) {
    tc_fence_after_sync();
    if constexpr (CG == 2) tmem_dealloc_pair(tmem_base, TMEM_COLS);
    else tmem_dealloc(tmem_base, TMEM_COLS);
  }
  if (threadIdx.x == 0) {                               // a kernel may run this body again (fused expert layer): leave no live barrier behind
    for (int i = 0; i < 2 * STAGES + 4; ++i) mbar_inval(&bars[i]);
  }
  __syncthreads();
  if constexpr (TP == TP_AG_GEMM) {
    // The last CTA of the grid tells every peer "my GEMM no longer reads my staging buffer" and waits for the
    // same from them: when this kernel ends, the next call may push into any peer's staging buffer.
    if (threadIdx.x == 0) {
      __threadfence();
      if (atomicAdd(tpp->done_ctr, 1u) == gridDim.x - 1) {
        *tpp->done_ctr = 0u;
        peer_handshake(*tpp, tp_epoch, 1, true, p.status);
        *tpp->epoch_ptr = tp_epoch;
      }
    }
  }
  if constexpr (TP == TP_GEMM_RS) {
    // ---------------------------------------------------------------- reduce-scatter half: handshake, then sum the slots
    const TpParams& tp = *tpp;
    __shared__ int s_go;
    if (threadIdx.x == 0) {
      s_go = 1;
      __threadfence_system();                                    // this CTA's peer stores are out
      if (atomicAdd(tp.done_ctr, 1u) == gridDim.x - 1) {
        *tp.done_ctr = 0u;
        const bool ok = peer_handshake(tp, tp_epoch, 1, true, p.status);   // every rank has stored all its partials
        __threadfence();
        *tp.epoch_ptr = tp_epoch;                                   // every CTA has read the old value long ago
        if (ok) st_release_gpu_u32(tp.go, tp_epoch);
      }
      if (!wait_flag<false>(tp.go, tp_epoch, 2 * tp.wait_cycles, p.status, ST_TIMEOUT_PEER_FLAG)) s_go = 0;
      __threadfence();
    }
    __syncthreads();
    if (s_go) {
      const long long rows_per_rank = (long long)tp.blocks_per_rank * BM;
      const long long n8 = rows_per_rank * p.N / 8;              // N % 8 == 0, ldc == N
      const __nv_bfloat16* slots = reinterpret_cast<const __nv_bfloat16*>(tp.slots_peer[tp.rank]) + (long long)(tp_epoch & 1u) * tp.world * rows_per_rank * p.N;
      const __nv_bfloat16* res = reinterpret_cast<const __nv_bfloat16*>(p.residual);
      __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(tp.out);
      for (long long i = (long long)blockIdx.x * GEMM_THREADS + threadIdx.x; i < n8; i += (long long)gridDim.x * GEMM_THREADS) {
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int r = 0; r < tp.world; ++r) {
          const uint4 u = __ldcg(reinterpret_cast<const uint4*>(slots + ((long long)r * rows_per_rank * p.N) + i * 8));   // written by peers: read at L2
          const float2 a0 = unpack_bf16x2(u.x), a1 = unpack_bf16x2(u.y), a2 = unpack_bf16x2(u.z), a3 = unpack_bf16x2(u.w);
          acc[0] += a0.x; acc[1] += a0.y; acc[2] += a1.x; acc[3] += a1.y; acc[4] += a2.x; acc[5] += a2.y; acc[6] += a3.x; acc[7] += a3.y;
        }
        if (res) {
          const long long row = (i * 8) / p.N, col = (i * 8) % p.N;
          const uint4 u = *reinterpret_cast<const uint4*>(res + row * p.ldr + col);
          const float2 a0 = unpack_bf16x2(u.x), a1 = unpack_bf16x2(u.y), a2 = unpack_bf16x2(u.z), a3 = unpack_bf16x2(u.w);
          acc[0] += a0.x; acc[1] += a0.y; acc[2] += a1.x; acc[3] += a1.y; acc[4] += a2.x; acc[5] += a2.y; acc[6] += a3.x; acc[7] += a3.y;
        }
        *reinterpret_cast<uint4*>(out + i * 8) = make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]),
                                                             pack_bf16x2(acc[4], acc[5]), pack_bf16x2(acc[6], acc[7]));
      }
    }
  }
}

template <typename T, int BN, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const __grid_constant__ GemmParams p,
            const __grid_constant__ OutMaps om) {
  gemm_body<T, BN, A_MN, B_MN, TP_NONE>(tmA, tmB, p, nullptr, &om);
}

// CTA-pair variant: bf16, 256 x 256 tile per pair, launched as clusters of two
template <bool A_MN, bool B_MN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const __grid_constant__ GemmParams p,
                 const __grid_constant__ OutMaps om) {
  gemm_body<__nv_bfloat16, 256, A_MN, B_MN, TP_NONE, 2>(tmA, tmB, p, nullptr, &om);
}

// ---------------------------------------------------------------------------- expert-parallel MoE layer, forward, ONE kernel
// dispatch (token rows stored into the owning rank's expert buffers over NVLink, slots claimed with remote atomics)
// -> cross-rank barrier -> grouped GEMM 1 (+bias, activation, saved pre-activation) over the real per-expert counts
// -> grid barrier -> grouped GEMM 2 into the peer-visible output buffer -> cross-rank barrier -> combine (weighted sum of
// the k expert rows of every token, read from the owners over NVLink) while the input buffer is saved for the backward
// and cleared -> cross-rank barrier. One persistent launch of one CTA per SM: the barriers inside it need every CTA
// resident. No host synchronisation, no NCCL; every wait is bounded by a clock budget and reports through the status word.
constexpr int MOEF_MAX_RANKS = 8;
struct MoeFusedArgs {
  const __nv_bfloat16* x; const int* idx; int* dest;        // [T, d], [T, k] expert ids, [T, k] global row ids (out)
  void* xbuf[MOEF_MAX_RANKS]; int* fill[MOEF_MAX_RANKS];     // every rank's expert input buffer [E_local, cap, d] and slot counters [E_local]
  const void* ybuf[MOEF_MAX_RANKS];                          // every rank's expert output buffer [E_local, cap, d]
  uint32_t* bar_flags[MOEF_MAX_RANKS];                       // cross-rank barrier flags (shared with the barrier kernel of the backward)
  uint32_t* bar_words;                                       // local: [0] cross-rank barriers passed so far
  uint32_t* sync;                                            // local: [0] CTA arrivals, [1] barrier generation
  const float* w; __nv_bfloat16* out;                        // [T, k] gate weights, [T, d] result
  __nv_bfloat16* xsave;                                      // copy of this rank's expert inputs for the weight gradient
  int* counts_out;                                           // [E_local] rows in use per local expert (for the backward)
  long long tokens, rows_per_rank, wait_cycles;
  int k, d, E_local, cap, rank, world;
  uint32_t* status;
};

__device__ __forceinline__ void moef_barrier(const MoeFusedArgs& a, uint32_t gen, uint32_t epoch, bool cross) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();                                  // this CTA's stores, peer stores included, are out
    const uint32_t old = atomicAdd(a.sync, 1u);
    if (old % gridDim.x == gridDim.x - 1) {                  // the last CTA to arrive speaks for the rank
      if (cross && a.world > 1) {
        for (int r = 0; r < a.world; ++r) st_release_sys_u32(a.bar_flags[r] + a.rank, epoch);
        for (int r = 0; r < a.world; ++r)
          if (!wait_flag<true>(a.bar_flags[a.rank] + r, epoch, a.wait_cycles, a.status, ST_TIMEOUT_PEER_FLAG)) break;
      }
      if (cross) { __threadfence_system(); a.bar_words[0] = epoch; }
      __threadfence();
      st_release_gpu_u32(a.sync + 1, gen);
    }
    wait_flag<false>(a.sync + 1, gen, 2 * a.wait_cycles, a.status, ST_TIMEOUT_GENERIC);
    __threadfence();
  }
  __syncthreads();
}

__global__ void __launch_bounds__(GEMM_THREADS, 1)
moe_fused_fwd_kernel(const __grid_constant__ CUtensorMap tmA1, const __grid_constant__ CUtensorMap tmB1, const __grid_constant__ GemmParams p1,
                     const __grid_constant__ OutMaps om1, const __grid_constant__ CUtensorMap tmA2, const __grid_constant__ CUtensorMap tmB2,
                     const __grid_constant__ GemmParams p2, const __grid_constant__ OutMaps om2, const __grid_constant__ MoeFusedArgs a) {
  const uint32_t gen0 = *reinterpret_cast<volatile const uint32_t*>(a.sync + 1);
  const uint32_t ep0 = *reinterpret_cast<volatile const uint32_t*>(a.bar_words);
  const int lane = threadIdx.x & 31;
  const long long warp_g = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5, n_warps = ((long long)gridDim.x * blockDim.x) >> 5;
  const long long row_vec = a.d / 8;                         // 16-byte vectors per row
  // ---- dispatch: one warp per (token, choice)
  for (long long wid = warp_g; wid < a.tokens * a.k; wid += n_warps) {
    const long long t = wid / a.k;
    const int e = a.idx[wid];
    const int owner = e / a.E_local, el = e % a.E_local;
    int slot = 0;
    if (lane == 0) slot = atomicAdd_system(a.fill[owner] + el, 1);
    slot = __shfl_sync(0xffffffffu, slot, 0);
    if (slot >= a.cap) { if (lane == 0) a.dest[wid] = -1; continue; }
    if (lane == 0) a.dest[wid] = (owner * a.E_local + el) * a.cap + slot;
    const uint4* src = reinterpret_cast<const uint4*>(a.x + t * a.d);
    uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(a.xbuf[owner]) + ((long long)el * a.cap + slot) * a.d);
    for (long long i = lane; i < row_vec; i += 32) dst[i] = src[i];
  }
  moef_barrier(a, gen0 + 1, ep0 + 1, true);                  // every rank's rows and slot counts have landed
  fence_proxy_async_all();                                   // ... and are visible to the TMA loads below
  gemm_body<__nv_bfloat16, 256, false, false, TP_NONE, 1, true>(tmA1, tmB1, p1, nullptr, &om1);
  moef_barrier(a, gen0 + 2, 0u, false);                      // all of h is written
  fence_proxy_async_all();
  gemm_body<__nv_bfloat16, 256, false, false, TP_NONE, 1>(tmA2, tmB2, p2, nullptr, &om2);
  moef_barrier(a, gen0 + 3, ep0 + 2, true);                  // every rank's expert outputs are in place
  // ---- combine: one warp per token; rows may live on a peer
  for (long long t = warp_g; t < a.tokens; t += n_warps) {
    for (long long c = lane; c < row_vec; c += 32) {
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      for (int j = 0; j < a.k; ++j) {
        const int r = a.dest[t * a.k + j];
        if (r < 0) continue;
        const float wj = a.w[t * a.k + j];
        const int owner = (int)(r / a.rows_per_rank);
        const long long lr = r % a.rows_per_rank;
        const uint4 v = __ldcg(reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(a.ybuf[owner]) + lr * a.d) + c);
        const __nv_bfloat162* hh = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
        for (int q = 0; q < 4; ++q) { const float2 f = __bfloat1622float2(hh[q]); acc[2 * q] += wj * f.x; acc[2 * q + 1] += wj * f.y; }
      }
      uint4 o;
      __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
      for (int q = 0; q < 4; ++q) oh[q] = __floats2bfloat162_rn(acc[2 * q], acc[2 * q + 1]);
      *(reinterpret_cast<uint4*>(a.out + t * a.d) + c) = o;
    }
  }
  // ---- keep the expert inputs for the weight gradient and clear the buffer for the next layer (rows in use, rounded up to
  //      the 128-row tiles the backward's K loop covers; rows past a count are zero already and are saved as zeros)
  {
    uint4* xb = reinterpret_cast<uint4*>(a.xbuf[a.rank]);
    uint4* xs = reinterpret_cast<uint4*>(a.xsave);
    const int* fill = a.fill[a.rank];
    const long long total_rows = (long long)a.E_local * a.cap;
    for (long long row = warp_g; row < total_rows; row += n_warps) {
      const int e = (int)(row / a.cap), r = (int)(row % a.cap);
      const int cnt = min(*reinterpret_cast<volatile const int*>(fill + e), a.cap);
      if (r >= (cnt + 127) / 128 * 128) continue;
      for (long long i = lane; i < row_vec; i += 32) {
        const uint4 v = xb[row * row_vec + i];
        if (xs) xs[row * row_vec + i] = v;
        xb[row * row_vec + i] = make_uint4(0u, 0u, 0u, 0u);
      }
    }
  }
  moef_barrier(a, gen0 + 4, 0u, false);                      // every CTA has read the slot counts
  if (blockIdx.x == 0)
    for (int e = threadIdx.x; e < a.E_local; e += blockDim.x) {
      int* f = a.fill[a.rank] + e;
      a.counts_out[e] = min(*reinterpret_cast<volatile int*>(f), a.cap);
      *f = 0;
    }
  moef_barrier(a, gen0 + 5, ep0 + 3, true);                  // peers have read my outputs; everyone's input buffers are clear
}

// bf16, K-major x K-major (the Linear forward layout) fused with its neighbouring collective
template <int BN, int TP>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_tp_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const __grid_constant__ GemmParams p,
               const __grid_constant__ TpParams tp, const __grid_constant__ PeerMaps pm) {
  gemm_body<__nv_bfloat16, BN, false, false, TP>(tmA, tmB, p, &tp, nullptr, &pm);
}

// ---------------------------------------------------------------------------- host side
template <typename T> struct DT;
template <> struct DT<__nv_bfloat16> { static constexpr CUtensorMapDataType v = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16; };
template <> struct DT<float> { static constexpr CUtensorMapDataType v = CU_TENSOR_MAP_DATA_TYPE_FLOAT32; };
template <> struct DT<s8s8_t> { static constexpr CUtensorMapDataType v = CU_TENSOR_MAP_DATA_TYPE_UINT8; };
template <> struct DT<u8s8_t> { static constexpr CUtensorMapDataType v = CU_TENSOR_MAP_DATA_TYPE_UINT8; };
template <> struct DT<e4m3_t> { static constexpr CUtensorMapDataType v = CU_TENSOR_MAP_DATA_TYPE_UINT8; };

// Opt in to the large dynamic shared-memory carve-out (once per instantiation).
template <typename T, int BN, bool A_MN, bool B_MN>
static int gemm_set_attr() {
  static bool done = false;
  if (done) return 0;
  (void)cudaGetLastError();   // do not inherit a stale error from an unrelated earlier call
  cudaError_t e = cudaFuncSetAttribute(gemm_kernel<T, BN, A_MN, B_MN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       GemmSmem<T, BN, A_MN, B_MN>::TOTAL);
  if (e != cudaSuccess) return (int)e;
  done = true;
  return 0;
}

static int g_tma_store = -1;     // -1: from the environment on first use (B200NN_GEMM_TMA_STORE=0 turns it off)
// Output maps for the bf16 store path; `use` stays 0 (plain stores) whenever a rule of the copy engine is not met.
static void make_out_maps(OutMaps& om, const GemmParams& p, int BN) {
  om.use = 0;
  if (g_tma_store < 0) { const char* e = getenv("B200NN_GEMM_TMA_STORE"); g_tma_store = (e && e[0] == '0') ? 0 : 1; }
  if (!g_tma_store || p.out_mode != OUT_BF16 || !p.vec_ok || BN < 128) return;
  const unsigned long long ldb = (unsigned long long)p.ldc * 2, sb = (unsigned long long)p.strideC * 2;
  if (ldb % 16 || (p.batch > 1 && sb % 16) || (reinterpret_cast<uintptr_t>(p.C) & 15)) return;
  if (make_tmap_3d(&om.c, p.C, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, p.N, p.M, p.batch, ldb, sb, 64, 32, CU_TENSOR_MAP_SWIZZLE_128B)) return;
  om.aux = om.c;
  if (p.aux_out) {
    if (reinterpret_cast<uintptr_t>(p.aux_out) & 15) return;
    if (make_tmap_3d(&om.aux, p.aux_out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, p.N, p.M, p.batch, ldb, sb, 64, 32, CU_TENSOR_MAP_SWIZZLE_128B)) return;
  }
  om.use = 1;
}

template <typename T, int BN, bool A_MN, bool B_MN>
static int launch_one(const GemmArgs& a, cudaStream_t stream, int num_sms) {
  using S = GemmSmem<T, BN, A_MN, B_MN>;
  constexpr int BK = S::BK;
  constexpr int ATOM = TILE_K_BYTES / sizeof(T);
  CUtensorMap tmA, tmB;
  int rc;
  // K-major: view [batch][rows][K], box {BK, rows_per_tile}. MN-major: view [batch][K][rows], box {ATOM, BK}.
  if (!A_MN) rc = make_tmap_3d(&tmA, a.A, DT<T>::v, sizeof(T), a.K, a.M, a.batch, a.lda * sizeof(T), a.strideA * sizeof(T), BK, BM, CU_TENSOR_MAP_SWIZZLE_128B);
  else       rc = make_tmap_3d(&tmA, a.A, DT<T>::v, sizeof(T), a.M, a.K, a.batch, a.lda * sizeof(T), a.strideA * sizeof(T), ATOM, BK, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return 100 + rc;
  if (!B_MN) rc = make_tmap_3d(&tmB, a.B, DT<T>::v, sizeof(T), a.K, a.N, a.batch, a.ldb * sizeof(T), a.strideB * sizeof(T), BK, BN, CU_TENSOR_MAP_SWIZZLE_128B);
  else       rc = make_tmap_3d(&tmB, a.B, DT<T>::v, sizeof(T), a.N, a.K, a.batch, a.ldb * sizeof(T), a.strideB * sizeof(T), ATOM, BK, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return 200 + rc;

  auto kfn = gemm_kernel<T, BN, A_MN, B_MN>;
  { int e = gemm_set_attr<T, BN, A_MN, B_MN>(); if (e) return 300 + e; }
  GemmParams p = a.p;
  const long long m_blocks = (p.M + BM - 1) / BM, n_blocks = (p.N + BN - 1) / BN;
  const long long tiles = m_blocks * n_blocks * p.splits * p.batch;
  int grid = (int)(tiles < num_sms ? tiles : num_sms);
  if (grid < 1) grid = 1;
  OutMaps om;
  om.c = tmA; om.aux = tmA;
  make_out_maps(om, p, BN);
  cudaError_t e = launch_pdl(kfn, dim3(grid), dim3(GEMM_THREADS), S::TOTAL, stream, tmA, tmB, p, om);
  if (e == cudaSuccess) e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}

static int g_pair_mode = -1;     // -1: from the environment on first use; 0: off; 1: where it pays; 2: wherever the shape allows
static bool pair_enabled() {
  if (g_pair_mode < 0) {
    const char* e = getenv("B200NN_GEMM_PAIR");
    g_pair_mode = (e && e[0] == '0') ? 0 : 1;
  }
  return g_pair_mode >= 1;
}

template <bool A_MN, bool B_MN>
static int pair_set_attr() {
  static bool done = false;
  if (done) return 0;
  (void)cudaGetLastError();
  cudaError_t e = cudaFuncSetAttribute(gemm_pair_kernel<A_MN, B_MN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       GemmSmem<__nv_bfloat16, 256, A_MN, B_MN, 2>::TOTAL);
  if (e != cudaSuccess) return (int)e;
  done = true;
  return 0;
}

// 256 x 256 tiles on CTA pairs. Worth it when there are enough pair tiles to fill the machine.
template <bool A_MN, bool B_MN>
static int launch_pair(const GemmArgs& a, cudaStream_t stream, int num_sms) {
  using T = __nv_bfloat16;
  using S = GemmSmem<T, 256, A_MN, B_MN, 2>;
  constexpr int BK = S::BK, BN = 256;
  constexpr int ATOM = TILE_K_BYTES / sizeof(T);
  CUtensorMap tmA, tmB;
  int rc;
  if (!A_MN) rc = make_tmap_3d(&tmA, a.A, DT<T>::v, sizeof(T), a.K, a.M, a.batch, a.lda * sizeof(T), a.strideA * sizeof(T), BK, BM, CU_TENSOR_MAP_SWIZZLE_128B);
  else       rc = make_tmap_3d(&tmA, a.A, DT<T>::v, sizeof(T), a.M, a.K, a.batch, a.lda * sizeof(T), a.strideA * sizeof(T), ATOM, BK, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return 100 + rc;
  if (!B_MN) rc = make_tmap_3d(&tmB, a.B, DT<T>::v, sizeof(T), a.K, a.N, a.batch, a.ldb * sizeof(T), a.strideB * sizeof(T), BK, BN / 2, CU_TENSOR_MAP_SWIZZLE_128B);
  else       rc = make_tmap_3d(&tmB, a.B, DT<T>::v, sizeof(T), a.N, a.K, a.batch, a.ldb * sizeof(T), a.strideB * sizeof(T), ATOM, BK, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return 200 + rc;
  { int e = pair_set_attr<A_MN, B_MN>(); if (e) return 300 + e; }
  GemmParams p = a.p;
  const long long m_blocks = (p.M + 2 * BM - 1) / (2 * BM), n_blocks = (p.N + BN - 1) / BN;
  const long long tiles = m_blocks * n_blocks * p.splits * p.batch;
  const long long pairs = num_sms / 2;
  int grid = 2 * (int)(tiles < pairs ? tiles : pairs);
  OutMaps om;
  om.c = tmA; om.aux = tmA;
  make_out_maps(om, p, BN);
  cudaError_t e = launch_pdl_cluster2(gemm_pair_kernel<A_MN, B_MN>, dim3(grid), dim3(GEMM_THREADS), S::TOTAL, stream, tmA, tmB, p, om);
  if (e == cudaSuccess) e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}

template <int BN, int TP>
static int launch_tp(const GemmArgs& a, const TpParams& tp, cudaStream_t stream, int num_sms) {
  using T = __nv_bfloat16;
  using S = GemmSmem<T, BN, false, false>;
  constexpr int BK = S::BK;
  CUtensorMap tmA, tmB;
  // A: TP_AG_GEMM multiplies out of the local staging copy [M, K]; TP_GEMM_RS out of the caller's A
  const void* aptr = (TP == TP_AG_GEMM) ? tp.stage_peer[tp.rank] : a.A;
  const long long lda = (TP == TP_AG_GEMM) ? a.K : a.lda;
  int rc = make_tmap_3d(&tmA, aptr, DT<T>::v, sizeof(T), a.K, a.M, 1, lda * sizeof(T), (long long)a.M * lda * sizeof(T), BK, BM, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return 100 + rc;
  rc = make_tmap_3d(&tmB, a.B, DT<T>::v, sizeof(T), a.K, a.N, 1, a.ldb * sizeof(T), (long long)a.N * a.ldb * sizeof(T), BK, BN, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return 200 + rc;
  static bool attr_done = false;
  if (!attr_done) {
    (void)cudaGetLastError();
    cudaError_t e = cudaFuncSetAttribute(gemm_tp_kernel<BN, TP>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
    if (e != cudaSuccess) return 300 + (int)e;
    attr_done = true;
  }
  // every CTA must be resident at once (CTAs wait on one another): one CTA per SM, grid <= SM count
  int grid = num_sms;
  if (TP == TP_AG_GEMM && grid - tp.copy_ctas < 1) return -6;
  PeerMaps pm;
  pm.use = 0;
  for (int r = 0; r < TP_MAX_WORLD; ++r) pm.m[r] = tmA;
  if (TP == TP_AG_GEMM) {
    static int tp_bulk = -1;
    if (tp_bulk < 0) { const char* e = getenv("B200NN_TP_BULK_GATHER"); tp_bulk = (e && e[0] == '0') ? 0 : 1; }
    if (tp_bulk && S::STAGE_BYTES >= 32 * 1024) pm.use = 2;
  }
  if (TP == TP_GEMM_RS && BN >= 128) {
    static int tp_tma = -1;
    if (tp_tma < 0) { const char* e = getenv("B200NN_TP_TMA_STORE"); tp_tma = (e && e[0] == '0') ? 0 : 1; }
    const unsigned long long rows_per_rank = (unsigned long long)tp.blocks_per_rank * BM, nb = (unsigned long long)a.p.N * 2;
    if (tp_tma && a.p.N % 8 == 0) {
      pm.use = 1;
      for (int r = 0; r < tp.world; ++r)
        if ((reinterpret_cast<uintptr_t>(tp.slots_peer[r]) & 15) ||
            make_tmap_3d(&pm.m[r], tp.slots_peer[r], DT<T>::v, sizeof(T), a.p.N, rows_per_rank, 2ull * tp.world, nb, rows_per_rank * nb, 64, 32,
                         CU_TENSOR_MAP_SWIZZLE_128B)) { pm.use = 0; break; }
    }
  }
  gemm_tp_kernel<BN, TP><<<grid, GEMM_THREADS, S::TOTAL, stream>>>(tmA, tmB, a.p, tp, pm);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}

template <typename T, int BN>
static int launch_major(const GemmArgs& a, cudaStream_t s, int sms) {
  if constexpr (BN == 256 && sizeof(T) == 2) {
    // CTA pairs when they occupy (nearly) as many SMs as the 128-row tiles would: a pair tile is two CTAs, so a split-K
    // weight gradient whose 128-row tiles were sized to fill the machine keeps its CTA count and moves a third less
    // operand traffic from L2 per FLOP
    const int sp = a.p.splits > 0 ? a.p.splits : 1;
    const long long pair_tiles = (long long)((a.p.M + 255) / 256) * ((a.p.N + 255) / 256) * sp * a.p.batch;
    const long long single_tiles = (long long)((a.p.M + 127) / 128) * ((a.p.N + 255) / 256) * sp * a.p.batch;
    const long long want = single_tiles < sms ? single_tiles : sms;
    // and the mainloop is long enough to matter (K >= 1024 per split: below that the tile is bound by its epilogue)
    const bool pays = 2 * pair_tiles * 100 >= want * 85 && a.K / sp >= 1024;
    if (pair_enabled() && a.p.M >= 256 && (pays || g_pair_mode == 2)) {
      if (!a.a_mn && !a.b_mn) return launch_pair<false, false>(a, s, sms);
      if (!a.a_mn && a.b_mn) return launch_pair<false, true>(a, s, sms);
      if (a.a_mn && !a.b_mn) return launch_pair<true, false>(a, s, sms);
      return launch_pair<true, true>(a, s, sms);
    }
  }
  if (!a.a_mn && !a.b_mn) return launch_one<T, BN, false, false>(a, s, sms);
  if (!a.a_mn && a.b_mn) return launch_one<T, BN, false, true>(a, s, sms);
  if (a.a_mn && !a.b_mn) return launch_one<T, BN, true, false>(a, s, sms);
  return launch_one<T, BN, true, true>(a, s, sms);
}

}  // namespace b200

// Loads every GEMM variant and sets its attributes up front (called once after the library is loaded).
extern "C" int b200_gemm_init() {
  using namespace b200;
  int e = 0;
#define B200_INIT_BN(BN) \
  e |= gemm_set_attr<__nv_bfloat16, BN, false, false>(); e |= gemm_set_attr<__nv_bfloat16, BN, false, true>(); \
  e |= gemm_set_attr<__nv_bfloat16, BN, true, false>(); e |= gemm_set_attr<__nv_bfloat16, BN, true, true>();
  B200_INIT_BN(64) B200_INIT_BN(128) B200_INIT_BN(256)
#undef B200_INIT_BN
  e |= pair_set_attr<false, false>(); e |= pair_set_attr<false, true>(); e |= pair_set_attr<true, false>(); e |= pair_set_attr<true, true>();
  e |= gemm_set_attr<float, 128, false, false>();
  e |= gemm_set_attr<s8s8_t, 128, false, false>(); e |= gemm_set_attr<s8s8_t, 256, false, false>();
  e |= gemm_set_attr<u8s8_t, 128, false, false>(); e |= gemm_set_attr<u8s8_t, 256, false, false>();
  e |= gemm_set_attr<e4m3_t, 128, false, false>(); e |= gemm_set_attr<e4m3_t, 256, false, false>();
  return e;
}

// 0: single-CTA tiles only; 1: 256 x 256 tiles on CTA pairs where they pay (default); 2: wherever M >= 256 and the tile is 256 wide
extern "C" int b200_gemm_set_pair(int mode) { b200::g_pair_mode = mode < 0 ? 0 : (mode > 2 ? 2 : mode); return 0; }

extern "C" int b200_gemm_set_tma_store(int on) { b200::g_tma_store = on ? 1 : 0; return 0; }

extern "C" int b200_gemm_launch(const b200::GemmArgs* args, int bn, int num_sms, cudaStream_t stream) {
  using namespace b200;
  const GemmArgs& a = *args;
  if (a.p.M <= 0 || a.p.N <= 0 || a.p.batch <= 0) return 0;
  if (a.dtype == GEMM_F32) {
    // TF32 runs K-major only: MN-major 32-bit operands need a different swizzle atom, so the
    // front-end hands this path explicitly transposed operands (b200_transpose).
    if (a.a_mn || a.b_mn) return -4;
    return launch_one<float, 128, false, false>(a, stream, num_sms);
  }
  if (a.dtype != GEMM_BF16) {
    // 8-bit operands: K-major only (weights are stored [N,K] once at quantisation time)
    if (a.a_mn || a.b_mn) return -4;
    if (a.p.out_mode == OUT_I32 && a.dtype == GEMM_E4M3) return -5;
    const bool wide = bn == 256;
    switch (a.dtype) {
      case GEMM_S8S8: return wide ? launch_one<s8s8_t, 256, false, false>(a, stream, num_sms) : launch_one<s8s8_t, 128, false, false>(a, stream, num_sms);
      case GEMM_U8S8: return wide ? launch_one<u8s8_t, 256, false, false>(a, stream, num_sms) : launch_one<u8s8_t, 128, false, false>(a, stream, num_sms);
      case GEMM_E4M3: return wide ? launch_one<e4m3_t, 256, false, false>(a, stream, num_sms) : launch_one<e4m3_t, 128, false, false>(a, stream, num_sms);
      default: return -3;
    }
  }
  switch (bn) {
    case 64: return launch_major<__nv_bfloat16, 64>(a, stream, num_sms);
    case 128: return launch_major<__nv_bfloat16, 128>(a, stream, num_sms);
    case 256: return launch_major<__nv_bfloat16, 256>(a, stream, num_sms);
    default: return -2;
  }
}

// Tensor-parallel GEMM (see TpParams). bf16 operands, both K-major, batch 1, no split-K, bf16 output.
extern "C" int b200_gemm_tp_launch(const b200::GemmArgs* args, const b200::TpParams* tp, int bn, int num_sms, cudaStream_t stream) {
  using namespace b200;
  const GemmArgs& a = *args;
  if (a.dtype != GEMM_BF16 || a.a_mn || a.b_mn || a.p.batch != 1 || a.p.splits != 1 || a.p.out_mode != OUT_BF16) return -3;
  if (tp->world < 1 || tp->world > TP_MAX_WORLD || tp->blocks_per_rank < 1 || a.p.M != tp->world * tp->blocks_per_rank * BM) return -7;
  if (a.p.K % 8 != 0 || a.p.N % 8 != 0) return -8;
  if (tp->mode == TP_AG_GEMM) {
    if (tp->world > 1 && tp->copy_ctas < 1) return -6;
    return bn == 256 ? launch_tp<256, TP_AG_GEMM>(a, *tp, stream, num_sms) : launch_tp<128, TP_AG_GEMM>(a, *tp, stream, num_sms);
  }
  if (tp->mode == TP_GEMM_RS) {
    if (a.p.ldc != a.p.N || !a.p.vec_ok || a.p.act != ACT_NONE || a.p.aux_out || a.p.aux_in) return -9;
    return bn == 256 ? launch_tp<256, TP_GEMM_RS>(a, *tp, stream, num_sms) : launch_tp<128, TP_GEMM_RS>(a, *tp, stream, num_sms);
  }
  return -2;
}

// One launch for the forward of an expert-parallel MoE layer (see moe_fused_fwd_kernel). g1 / g2 describe the two grouped
// GEMMs exactly as b200_gemm_launch would take them (bf16, both operands K-major, 256-wide tiles, no split-K, batch =
// local experts, m_valid = this rank's slot counters).
extern "C" int b200_moe_fused_fwd(const b200::GemmArgs* g1, const b200::GemmArgs* g2, const b200::MoeFusedArgs* fa, int num_sms, cudaStream_t stream) {
  using namespace b200;
  using T = __nv_bfloat16;
  using S = GemmSmem<T, 256, false, false>;
  constexpr int BK = S::BK, BN = 256;
  if (fa->world < 1 || fa->world > MOEF_MAX_RANKS || fa->d % 8) return -1;
  const GemmArgs* gs[2] = {g1, g2};
  CUtensorMap tmA[2], tmB[2];
  OutMaps om[2];
  for (int i = 0; i < 2; ++i) {
    const GemmArgs& a = *gs[i];
    if (a.dtype != GEMM_BF16 || a.a_mn || a.b_mn || a.p.splits != 1 || a.p.out_mode != OUT_BF16) return -3;
    int rc = make_tmap_3d(&tmA[i], a.A, DT<T>::v, sizeof(T), a.K, a.M, a.batch, a.lda * sizeof(T), a.strideA * sizeof(T), BK, BM, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return 100 + rc;
    rc = make_tmap_3d(&tmB[i], a.B, DT<T>::v, sizeof(T), a.K, a.N, a.batch, a.ldb * sizeof(T), a.strideB * sizeof(T), BK, BN, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return 200 + rc;
    om[i].c = tmA[i]; om[i].aux = tmA[i];
    make_out_maps(om[i], a.p, BN);
  }
  static bool attr_done = false;
  if (!attr_done) {
    (void)cudaGetLastError();
    cudaError_t e = cudaFuncSetAttribute(moe_fused_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
    if (e != cudaSuccess) return 300 + (int)e;
    attr_done = true;
  }
  // every CTA must be resident at once (CTAs wait on one another): one CTA per SM, grid = SM count, the same for every launch
  moe_fused_fwd_kernel<<<num_sms, GEMM_THREADS, S::TOTAL, stream>>>(tmA[0], tmB[0], g1->p, om[0], tmA[1], tmB[1], g2->p, om[1], *fa);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}
