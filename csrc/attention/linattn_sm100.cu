// A3 / A4: causal linear attention, forward and backward, as fused chunk kernels on tcgen05 / TMEM (sm_100a).
//
//   out_t = phi(s q_t) . S_t / (phi(s q_t) . z_t + eps),   S_t = sum_{u<=t} phi(s k_u) (x) v_u,   z_t = sum_{u<=t} phi(s k_u)
//
// with phi = ELU + 1 or ReLU^2 (rust-nn src/linear_attention.rs:42-94). The reference runs the causal form as a
// per-token rank-1 recurrence and its backward stores every S_t (src/linear_attention.rs:214-266, 502-632). Here one
// CTA owns one (batch, head) and walks its sequence in chunks of 128 tokens; thread t owns token t of the chunk (= TMEM
// lane t). Per chunk, with Q~ = phi(sQ), K~ = phi(sK) formed in shared memory in place on the TMA tiles:
//
//   forward     A = mask(Q~ K~^T)            NUM = Q~ S + A V          den = rowsum(A) + Q~ . z        out = NUM / (den + eps)
//               S += K~^T V                  z += colsum(K~)
//   backward 1  (same direction, carries S, z again)      G = dO / D,  dden = -(dO . O) / D
//               dA = mask(G V^T + dden 1^T)  dQ~ = dA K~ + G S^T + dden (x) z
//   backward 2  (reverse direction, carries dS = sum_later Q~^T G and dz = sum_later Q~^T dden)
//               dV = mask(A)^T G + K~ dS     dK~ = mask(dA)^T Q~ + V dS^T + 1 (x) dz
//               dS += Q~^T G                 dz += Q~^T dden
//   then dQ = s phi'(sQ) dQ~, dK = s phi'(sK) dK~ in the epilogue.
//
// Every product is a tcgen05.mma with fp32 accumulation in TMEM. The running state stays in TMEM in fp32 for the whole
// sequence; where it enters a product as an operand it is written to shared memory as TWO bf16 tiles (value and
// rounding remainder) and multiplied twice, so the state contributes ~16 mantissa bits: dQ is a difference of two
// nearly equal terms (G S^T against dden z) and a single bf16 copy of S loses it. z and dz are applied in fp32 by the
// threads. The same natural [d_k][d_v] tile serves as MN-major B operand (x S) and as K-major B operand (x S^T).
// No state is ever stored per token or per chunk: both backward kernels recompute what they need from Q, K, V, dO, O
// and the saved denominators.
//
// `s_in` / `s_out` (optional) are the state before the first token and after the last one; a sequence-parallel rank
// passes the sum of the lower ranks' states in and hands its own total out. Every wait is bounded (status word).
#include "../common/ptx.cuh"
#include "../common/tensormap.h"
#include "flash_sm100.h"

namespace b200 {

constexpr int LA_C = 128;                    // tokens per chunk = rows of every product = TMEM lanes

// Sequence-parallel exchange of the slice totals, done by the attention kernels themselves over NVLink peer memory.
// The state pass of a rank (role 1) writes its total into its OWN symmetric buffer and then raises one flag per
// (consumer rank, batch x head); the main pass (role 2) of a consumer waits for the flags of the ranks it depends on,
// pulls their totals with plain peer loads in rank order (so every run sums in the same order), keeps the sum in
// `prefix` and acknowledges. A total is double-buffered by call parity and is only overwritten once every consumer has
// acknowledged the call two earlier. The call counter is a device word that the last CTA of the main pass advances,
// so a captured graph replays with fresh epochs. All waits are bounded.
constexpr int LA_MAX_WORLD = 8;
struct LaExchange {
  float* state[LA_MAX_WORLD];       // every rank's totals [2][B*H][hd*hd + hd] fp32 (peer-mapped)
  uint32_t* flags[LA_MAX_WORLD];    // every rank's arrival flags [world][B*H] (peer-mapped): flags[c][r * BH + bh] = epoch
  uint32_t* acks[LA_MAX_WORLD];     // every rank's release flags [world][B*H] (peer-mapped): acks[r][c * BH + bh] = epoch
  float* prefix;                    // local [B*H][hd*hd + hd]: the sum the main pass started from (the backward needs it again)
  uint32_t* words;                  // local: [0] calls so far, [1] retired CTAs of the main pass
  long long wait_cycles;
  int rank, world;                  // world <= 1: no exchange
  int dir;                          // 0: sum over the LOWER ranks (forward states), 1: over the HIGHER ranks (backward)
  int role;                         // 0: none, 1: publish this slice's total, 2: consume
};

struct LinAttnArgs {
  AttnTensor q, k, v, o;                     // bf16 [B, S, H, hd] (any strides, hd contiguous)
  AttnTensor dout, dq, dk, dv;               // backward
  AttnTensor o_lo;                           // optional bf16 remainder O - bf16(O): written by forward, read by backward.
                                             // dden = -(dO . O) / D is one half of a difference of nearly equal terms
                                             // (S^T G against (G . O) z); 8 mantissa bits of O are not enough for it
  float* den;                                // [B, H, S] fp32: denominators incl. eps (written by forward, read by backward)
  const float* s_in;                         // optional [B*H][hd*hd + hd] fp32: state (row-major [d_k][d_v]) then z
  float* s_out;                              // optional, same layout: state after the last token (forward / state pass)
  const float* ds_in;                        // backward 2, optional: dS, dz flowing in from the tokens after this slice
  float* ds_out;                             // backward 2, optional: dS, dz at the first token (for the slices before it)
  int B, H, S, hd;
  float scale, eps;
  int kind;                                  // 0: ELU + 1, 1: ReLU^2
  int state_only;                            // forward: only accumulate the state (reads K, V; writes s_out)
  uint32_t* status;
  LaExchange sx;
};

__device__ __forceinline__ bool la_wait_flag(const uint32_t* f, uint32_t want, long long budget, uint32_t* status) {
  const long long t0 = clock64();
  for (;;) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
    if ((int32_t)(v - want) >= 0) return true;
    if (clock64() - t0 > budget) { if (status) atomicCAS(status, 0u, (uint32_t)ST_TIMEOUT_PEER_FLAG); return false; }
    __nanosleep(64);
  }
}
__device__ __forceinline__ void la_set_flag(uint32_t* f, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(f), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t la_epoch(const LinAttnArgs& p) {
  return (p.sx.role != 0 && p.sx.world > 1) ? *reinterpret_cast<volatile const uint32_t*>(p.sx.words) + 1u : 0u;
}
// Main pass: the state this (batch, head) starts from. Without an exchange that is `fallback` (the caller's s_in / ds_in).
template <int HD>
__device__ __forceinline__ const float* la_consume(const LinAttnArgs& p, int bh, uint32_t epoch, const float* fallback) {
  const LaExchange& x = p.sx;
  if (x.role != 2 || x.world <= 1) return fallback;
  const int lo = x.dir == 0 ? 0 : x.rank + 1, hi = x.dir == 0 ? x.rank : x.world;       // the ranks whose totals flow in
  if (lo >= hi) return nullptr;
  constexpr int ST = HD * HD + HD;
  const int BH = p.B * p.H, tid = threadIdx.x;
  int good = 1;
  if (tid >= lo && tid < hi && !la_wait_flag(x.flags[x.rank] + (size_t)tid * BH + bh, epoch, x.wait_cycles, p.status)) good = 0;
  const bool ok = __syncthreads_and(good) != 0;
  float4* dst = reinterpret_cast<float4*>(x.prefix + (size_t)bh * ST);
  for (int i = tid; i < ST / 4; i += blockDim.x) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int r = lo; r < hi && ok; ++r) {
      const float4 v = __ldcv(reinterpret_cast<const float4*>(x.state[r] + ((size_t)(epoch & 1u) * BH + bh) * ST) + i);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    dst[i] = acc;
  }
  __threadfence_system();
  __syncthreads();
  if (tid >= lo && tid < hi) la_set_flag(x.acks[tid] + (size_t)x.rank * BH + bh, epoch);        // "I have read your total"
  return x.prefix;
}
// State pass: where this slice's totals go. With an exchange: this rank's symmetric buffer (after the consumers of the
// call two earlier have released it); `la_publish_end` then raises the flags at the consumers.
template <int HD>
__device__ __forceinline__ float* la_publish_begin(const LinAttnArgs& p, int bh, uint32_t epoch, float* fallback) {
  const LaExchange& x = p.sx;
  if (x.role != 1 || x.world <= 1) return fallback;
  constexpr int ST = HD * HD + HD;
  const int BH = p.B * p.H, tid = threadIdx.x;
  const int lo = x.dir == 0 ? x.rank + 1 : 0, hi = x.dir == 0 ? x.world : x.rank;       // the ranks that will read it
  if (tid >= lo && tid < hi) la_wait_flag(x.acks[x.rank] + (size_t)tid * BH + bh, epoch - 2u, x.wait_cycles, p.status);
  __syncthreads();
  return x.state[x.rank] + (size_t)(epoch & 1u) * BH * ST;
}
__device__ __forceinline__ void la_publish_end(const LinAttnArgs& p, int bh, uint32_t epoch) {
  const LaExchange& x = p.sx;
  if (x.role != 1 || x.world <= 1) return;
  const int BH = p.B * p.H, tid = threadIdx.x;
  const int lo = x.dir == 0 ? x.rank + 1 : 0, hi = x.dir == 0 ? x.world : x.rank;
  __threadfence_system();
  __syncthreads();
  if (tid >= lo && tid < hi) la_set_flag(x.flags[tid] + (size_t)x.rank * BH + bh, epoch);
}
// Main pass, last thing: the last CTA to get here advances the call counter.
__device__ __forceinline__ void la_retire(const LinAttnArgs& p, uint32_t epoch) {
  const LaExchange& x = p.sx;
  if (x.role != 2 || x.world <= 1 || threadIdx.x != 0) return;
  __threadfence();
  if (atomicAdd(x.words + 1, 1u) == gridDim.x - 1) { x.words[1] = 0u; __threadfence(); x.words[0] = epoch; }
}

__device__ __forceinline__ float la_phi(float x, int kind) { return kind == 0 ? (x > 0.f ? x + 1.f : __expf(x)) : (x > 0.f ? x * x : 0.f); }
// derivative of phi expressed through its value: ELU+1: 1 for x > 0 (phi > 1) else phi; ReLU^2: 2 sqrt(phi)
__device__ __forceinline__ float la_dphi_from_phi(float p, int kind) { return kind == 0 ? (p > 1.f ? 1.f : p) : 2.f * sqrtf(p); }

// phi(scale * x) in place on a [128 rows][HD] bf16 tile of 128-byte-swizzled 64-column atoms; thread = row.
// Rows at or beyond `valid` become zero (TMA fills them with zeros, and phi(0) is 1 for ELU + 1).
template <int HD>
__device__ __forceinline__ void la_phi_tile(uint8_t* tile, int row, int valid, float scale, int kind) {
#pragma unroll
  for (int a = 0; a < HD / 64; ++a)
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      uint4* p = reinterpret_cast<uint4*>(tile + a * (LA_C * 128) + sw128_offset(row, c));
      uint4 u = *p;
      uint32_t* w = &u.x;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = unpack_bf16x2(w[j]);
        w[j] = row < valid ? pack_bf16x2(la_phi(f.x * scale, kind), la_phi(f.y * scale, kind)) : 0u;
      }
      *p = u;
    }
}

// fp32 row of a tile (thread = row) -> registers
template <int HD>
__device__ __forceinline__ void la_read_row(const uint8_t* tile, int row, float* out) {
#pragma unroll
  for (int a = 0; a < HD / 64; ++a)
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      const uint4 u = *reinterpret_cast<const uint4*>(tile + a * (LA_C * 128) + sw128_offset(row, c));
      const uint32_t* w = &u.x;
#pragma unroll
      for (int j = 0; j < 4; ++j) { const float2 f = unpack_bf16x2(w[j]); out[a * 64 + c * 8 + 2 * j] = f.x; out[a * 64 + c * 8 + 2 * j + 1] = f.y; }
    }
}

// column sums of a tile: thread k (< HD) returns sum over the 128 rows of element (row, k)
template <int HD>
__device__ __forceinline__ float la_colsum(const uint8_t* tile, int k) {
  const uint8_t* base = tile + (k >> 6) * (LA_C * 128) + (k & 7) * 2;
  const int chunk = (k & 63) >> 3;
  float s0 = 0.f, s1 = 0.f;
#pragma unroll 8
  for (int r = 0; r < LA_C; r += 2) {
    s0 += __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(base + sw128_offset(r, chunk)));
    s1 += __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(base + sw128_offset(r + 1, chunk)));
  }
  return s0 + s1;
}
// weighted column sums: sum_r w[r] * tile(r, k)
template <int HD>
__device__ __forceinline__ float la_colsum_w(const uint8_t* tile, int k, const float* w) {
  const uint8_t* base = tile + (k >> 6) * (LA_C * 128) + (k & 7) * 2;
  const int chunk = (k & 63) >> 3;
  float s0 = 0.f, s1 = 0.f;
#pragma unroll 8
  for (int r = 0; r < LA_C; r += 2) {
    s0 += w[r] * __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(base + sw128_offset(r, chunk)));
    s1 += w[r + 1] * __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(base + sw128_offset(r + 1, chunk)));
  }
  return s0 + s1;
}

// One fp32 row of HD values -> bf16 "value" tile and bf16 "remainder" tile (row = thread), [rows][HD] swizzled atoms
// of `rows` rows each.
template <int HD>
__device__ __forceinline__ void la_write_hilo(uint8_t* hi, uint8_t* lo, int rows, int row, const float* v) {
#pragma unroll
  for (int g = 0; g < HD / 8; ++g) {
    uint32_t h[4], l[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float a = v[g * 8 + 2 * j], b = v[g * 8 + 2 * j + 1];
      const __nv_bfloat16 ah = __float2bfloat16_rn(a), bh = __float2bfloat16_rn(b);
      h[j] = pack_bf16x2(__bfloat162float(ah), __bfloat162float(bh));
      l[j] = pack_bf16x2(a - __bfloat162float(ah), b - __bfloat162float(bh));
    }
    const uint32_t off = (g >> 3) * (rows * 128) + sw128_offset(row, g & 7);
    *reinterpret_cast<uint4*>(hi + off) = make_uint4(h[0], h[1], h[2], h[3]);
    *reinterpret_cast<uint4*>(lo + off) = make_uint4(l[0], l[1], l[2], l[3]);
  }
}

// fp32 row of 128 values -> bf16 K-major [128][128] tile (two atoms), row = thread
__device__ __forceinline__ void la_write_row128(uint8_t* tile, int row, const float* v) {
#pragma unroll
  for (int g = 0; g < 16; ++g) {
    const uint4 o = make_uint4(pack_bf16x2(v[g * 8], v[g * 8 + 1]), pack_bf16x2(v[g * 8 + 2], v[g * 8 + 3]),
                               pack_bf16x2(v[g * 8 + 4], v[g * 8 + 5]), pack_bf16x2(v[g * 8 + 6], v[g * 8 + 7]));
    *reinterpret_cast<uint4*>(tile + (g >> 3) * (LA_C * 128) + sw128_offset(row, g & 7)) = o;
  }
}

// fp32 row of 128 values -> bf16 value tile and bf16 remainder tile (both K-major [128][128]), row = thread
// (`with_lo` false: the value tile only)
__device__ __forceinline__ void la_write_row128_hilo(uint8_t* hi, uint8_t* lo, int row, const float* v, bool with_lo) {
#pragma unroll
  for (int g = 0; g < 16; ++g) {
    uint32_t h[4], l[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float a = v[g * 8 + 2 * j], b = v[g * 8 + 2 * j + 1];
      h[j] = pack_bf16x2(a, b);
      const float2 r = unpack_bf16x2(h[j]);
      l[j] = pack_bf16x2(a - r.x, b - r.y);
    }
    const uint32_t off = (g >> 3) * (LA_C * 128) + sw128_offset(row, g & 7);
    *reinterpret_cast<uint4*>(hi + off) = make_uint4(h[0], h[1], h[2], h[3]);
    if (with_lo) *reinterpret_cast<uint4*>(lo + off) = make_uint4(l[0], l[1], l[2], l[3]);
  }
}

template <int N>
__device__ __forceinline__ void la_tmem_row(uint32_t taddr, float* out) {
#pragma unroll
  for (int c = 0; c < N / 32; ++c) tmem_ld_x32(taddr + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&out[c * 32]));
  tmem_ld_wait();
}

// ---- MMA issue helpers (one thread). All tiles: atoms of 64 columns, 128-byte rows, 128-byte swizzle.
// D[128 x 128] = X Y^T, both operands K-major [128][HD]
template <int HD>
__device__ __forceinline__ void la_mma_xyT(uint32_t d, const uint8_t* x, const uint8_t* y) {
  constexpr uint32_t idesc = make_idesc(128, 128, CFMT_F32, FMT_BF16, FMT_BF16, 0, 0);
  const uint32_t lx = sdesc_lo(smem_u32(x), 0), ly = sdesc_lo(smem_u32(y), 0);
#pragma unroll
  for (int k = 0; k < HD / 16; ++k) {
    const uint32_t adv = (k >> 2) * (LA_C * 128) + (k & 3) * 32;
    umma_f16(d, sdesc_at<1024>(lx, adv), sdesc_at<1024>(ly, adv), idesc, k > 0);
  }
}
// D[128 x HD] (+)= P W with P K-major [128][KT] (KT = 128 tokens or HD) and W MN-major: [KT rows][HD], atoms `w_lbo` apart
template <int HD, int KT>
__device__ __forceinline__ void la_mma_pw(uint32_t d, const uint8_t* p, const uint8_t* w, uint32_t w_lbo, bool acc) {
  constexpr uint32_t idesc = make_idesc(128, HD, CFMT_F32, FMT_BF16, FMT_BF16, 0, 1);
  const uint32_t lp = sdesc_lo(smem_u32(p), 0), lw = sdesc_lo(smem_u32(w), w_lbo);
#pragma unroll
  for (int k = 0; k < KT / 16; ++k) {
    const uint32_t advp = (k >> 2) * (LA_C * 128) + (k & 3) * 32;
    umma_f16(d, sdesc_at<1024>(lp, advp), sdesc_at<1024>(lw, k * 2048), idesc, acc || k > 0);
  }
}
// D[128 x HD] (+)= X W^T with X K-major [128][HD] and W K-major [HD rows][HD] (atoms of HD rows)
template <int HD>
__device__ __forceinline__ void la_mma_xwT(uint32_t d, const uint8_t* x, const uint8_t* w, bool acc) {
  constexpr uint32_t idesc = make_idesc(128, HD, CFMT_F32, FMT_BF16, FMT_BF16, 0, 0);
  const uint32_t lx = sdesc_lo(smem_u32(x), 0), lw = sdesc_lo(smem_u32(w), 0);
#pragma unroll
  for (int k = 0; k < HD / 16; ++k) {
    const uint32_t advx = (k >> 2) * (LA_C * 128) + (k & 3) * 32, advw = (k >> 2) * (HD * 128) + (k & 3) * 32;
    umma_f16(d, sdesc_at<1024>(lx, advx), sdesc_at<1024>(lw, advw), idesc, acc || k > 0);
  }
}
// State update D[128 (d_k, zero-padded) x HD] (+)= X^T W over the 128 tokens: X, W MN-major [128 tokens][HD].
// `x_lbo` is the distance from X's first 64-column atom to the next one; for HD = 64 it points at a tile of zeros, so
// that the product has the 128 rows the instruction wants and rows 64..127 of D stay zero.
template <int HD>
__device__ __forceinline__ void la_mma_xTw(uint32_t d, const uint8_t* x, uint32_t x_lbo, const uint8_t* w, bool acc) {
  constexpr uint32_t idesc = make_idesc(128, HD, CFMT_F32, FMT_BF16, FMT_BF16, 1, 1);
  const uint32_t lx = sdesc_lo(smem_u32(x), x_lbo), lw = sdesc_lo(smem_u32(w), LA_C * 128);
#pragma unroll
  for (int k = 0; k < LA_C / 16; ++k)
    umma_f16(d, sdesc_at<1024>(lx, k * 2048), sdesc_at<1024>(lw, k * 2048), idesc, acc || k > 0);
}

template <int HD>
struct LaSmem {
  static constexpr int TILE = LA_C * HD * 2;          // one [128][HD] operand tile
  static constexpr int PT = LA_C * LA_C * 2;          // one [128][128] tile
  static constexpr int ST = HD * HD * 2;              // one state tile [HD][HD]
  static constexpr int ZERO = HD == 64 ? TILE : 0;    // zero atom that pads the state update to 128 rows
  // The masked [128][128] tile of a chunk (A in the forward, dA in the dQ kernel) enters its product as value + remainder
  // like the state does: dQ is a difference of nearly equal sums, and one bf16 copy of the tile costs it ~2 % each way.
  // With head_dim 64 the remainder tile has its own buffer; with 128 (shared memory is full) it reuses the tile of the
  // operand that is dead by then (Q~ in the forward, G in the dQ kernel).
  static constexpr int PLO = HD == 64 ? PT : 0;
};

// ---------------------------------------------------------------------------------------------------- forward
// Thread mapping of the forward kernel: 8 warps. Warp w owns tile rows / TMEM lanes 32 (w & 3) .. + 31 (the lanes a warp
// may read) and column half w >> 2 of every row, so the elementwise work of a chunk is spread over twice the warps of a
// row-per-thread mapping and every scheduler has two warps to switch between (the kernel is bound by instruction
// latency, not by the tensor core: 4 k instructions per chunk and thread at ~5 cycles each with one warp per scheduler).
constexpr int LA_FWD_THREADS = 256;

// phi(scale * x) in place on this thread's half of its row (4 of the 8 16-byte chunks of every 64-column atom)
template <int HD>
__device__ __forceinline__ void la_phi_half(uint8_t* tile, int row, int hf, int valid, float scale, int kind) {
#pragma unroll
  for (int a = 0; a < HD / 64; ++a)
#pragma unroll
    for (int c4 = 0; c4 < 4; ++c4) {
      const int c = hf * 4 + c4;
      uint4* p = reinterpret_cast<uint4*>(tile + a * (LA_C * 128) + sw128_offset(row, c));
      uint4 u = *p;
      uint32_t* w = &u.x;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = unpack_bf16x2(w[j]);
        w[j] = row < valid ? pack_bf16x2(la_phi(f.x * scale, kind), la_phi(f.y * scale, kind)) : 0u;
      }
      *p = u;
    }
}
// this thread's half of (row . z)
template <int HD>
__device__ __forceinline__ float la_dot_half(const uint8_t* tile, int row, int hf, const float* z) {
  float acc0 = 0.f, acc1 = 0.f;
#pragma unroll
  for (int a = 0; a < HD / 64; ++a)
#pragma unroll
    for (int c4 = 0; c4 < 4; ++c4) {
      const int c = hf * 4 + c4;
      const uint4 u = *reinterpret_cast<const uint4*>(tile + a * (LA_C * 128) + sw128_offset(row, c));
      const uint32_t* w = &u.x;
      const float* zz = z + a * 64 + c * 8;
#pragma unroll
      for (int j = 0; j < 4; ++j) { const float2 f = unpack_bf16x2(w[j]); acc0 = fmaf(f.x, zz[2 * j], acc0); acc1 = fmaf(f.y, zz[2 * j + 1], acc1); }
    }
  return acc0 + acc1;
}
// 64 fp32 values = columns 64 hf .. of this thread's row of a [128][128] tile (atom hf) -> value and remainder tiles
__device__ __forceinline__ void la_write_half128_hilo(uint8_t* hi, uint8_t* lo, int row, int hf, const float* v, bool with_lo) {
#pragma unroll
  for (int g = 0; g < 8; ++g) {
    uint32_t h[4], l[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float a = v[g * 8 + 2 * j], b = v[g * 8 + 2 * j + 1];
      h[j] = pack_bf16x2(a, b);
      const float2 r = unpack_bf16x2(h[j]);
      l[j] = pack_bf16x2(a - r.x, b - r.y);
    }
    const uint32_t off = hf * (LA_C * 128) + sw128_offset(row, g);
    *reinterpret_cast<uint4*>(hi + off) = make_uint4(h[0], h[1], h[2], h[3]);
    if (with_lo) *reinterpret_cast<uint4*>(lo + off) = make_uint4(l[0], l[1], l[2], l[3]);
  }
}
// HD / 2 fp32 values = columns (HD / 2) hf .. of a state row -> value and remainder tiles ([rows][HD], atoms of `rows` rows)
template <int HD>
__device__ __forceinline__ void la_write_hilo_half(uint8_t* hi, uint8_t* lo, int rows, int row, int hf, const float* v) {
#pragma unroll
  for (int gg = 0; gg < HD / 16; ++gg) {
    const int g = hf * (HD / 16) + gg;
    uint32_t h[4], l[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float a = v[gg * 8 + 2 * j], b = v[gg * 8 + 2 * j + 1];
      h[j] = pack_bf16x2(a, b);
      const float2 r = unpack_bf16x2(h[j]);
      l[j] = pack_bf16x2(a - r.x, b - r.y);
    }
    const uint32_t off = (g >> 3) * (rows * 128) + sw128_offset(row, g & 7);
    *reinterpret_cast<uint4*>(hi + off) = make_uint4(h[0], h[1], h[2], h[3]);
    *reinterpret_cast<uint4*>(lo + off) = make_uint4(l[0], l[1], l[2], l[3]);
  }
}
// partial column sum: rows [r0, r0 + n) of column k
__device__ __forceinline__ float la_colsum_rows(const uint8_t* tile, int k, int r0, int n) {
  const uint8_t* base = tile + (k >> 6) * (LA_C * 128) + (k & 7) * 2;
  const int chunk = (k & 63) >> 3;
  float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll 4
  for (int r = r0; r < r0 + n; r += 4) {
    s0 += __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(base + sw128_offset(r, chunk)));
    s1 += __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(base + sw128_offset(r + 1, chunk)));
    s2 += __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(base + sw128_offset(r + 2, chunk)));
    s3 += __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(base + sw128_offset(r + 3, chunk)));
  }
  return (s0 + s1) + (s2 + s3);
}

template <int HD>
__global__ void __launch_bounds__(LA_FWD_THREADS, 1)
linattn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, const LinAttnArgs p) {
  using L = LaSmem<HD>;
  constexpr int KA = HD / 64;
  constexpr int HH = HD / 2;                  // columns of a HD-wide row per thread
  constexpr int ZP = LA_FWD_THREADS / HD;     // row groups of the column sums of K~ (4 or 2)
  constexpr uint32_t COL_A = 0, COL_NUM = 128, COL_S = 256;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + L::TILE;                 // 2 stages
  uint8_t* sZero = sK + 2 * L::TILE;          // HD = 64 only
  uint8_t* sV = sZero + L::ZERO;
  uint8_t* sP = sV + L::TILE;
  uint8_t* sShi = sP + L::PT;
  uint8_t* sSlo = sShi + L::ST;
  uint8_t* sPlo = HD == 64 ? sSlo + L::ST : sQ;
  float* sz = reinterpret_cast<float*>(sSlo + L::ST + L::PLO);      // [HD]
  float* s_part = sz + HD;                    // [2][128]: the halves' shares of a row's denominator
  float* s_zk = s_part + 2 * LA_C;            // [ZP][HD]: partial column sums of K~
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_zk + LA_FWD_THREADS);
  uint64_t* q_bar = bars; uint64_t* k_bar = bars + 1; uint64_t* v_bar = bars + 3; uint64_t* a_bar = bars + 4; uint64_t* b_bar = bars + 5;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 6);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int quad = warp & 3, hf = warp >> 2, row = quad * 32 + lane;
  const int bh = blockIdx.x, b = bh / p.H, h = bh % p.H;
  const int n_chunks = (p.S + LA_C - 1) / LA_C;
  const bool full = !p.state_only;
  // ELU + 1 features sit near 1, where a bf16 copy of the masked tile loses what the later subtraction needs; ReLU^2
  // features are spread over the exponent range and a single copy is enough (0.3 % measured)
  const bool rem = p.kind == 0;
  if ((smem_u32(smem) & 1023u) != 0) { if (tid == 0 && p.status) atomicCAS(p.status, 0u, (uint32_t)ST_BAD_ARGUMENT); return; }
  if (tid == 0) {
    mbar_init(q_bar, 1); mbar_init(&k_bar[0], 1); mbar_init(&k_bar[1], 1); mbar_init(v_bar, 1); mbar_init(a_bar, 1); mbar_init(b_bar, 1);
    fence_barrier_init();
    tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
  }
  if (warp == 0) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  if (HD == 64) for (int i = tid; i < L::ZERO / 16; i += LA_FWD_THREADS) reinterpret_cast<uint4*>(sZero)[i] = make_uint4(0, 0, 0, 0);
  // state before the first token: TMEM (fp32) and the two bf16 operand tiles
  const size_t st_stride = (size_t)HD * HD + HD;
  const uint32_t sx_epoch = la_epoch(p);
  const float* s_in = la_consume<HD>(p, bh, sx_epoch, p.s_in);       // the caller's state, or the lower ranks' totals
  if (tid < HD) {
    float s0[HD];
#pragma unroll
    for (int i = 0; i < HD; ++i) s0[i] = s_in ? s_in[bh * st_stride + (size_t)tid * HD + i] : 0.f;
    la_write_hilo<HD>(sShi, sSlo, HD, tid, s0);
    sz[tid] = s_in ? s_in[bh * st_stride + (size_t)HD * HD + tid] : 0.f;
  }
  tc_fence_before_sync();
  fence_proxy_async_smem();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t trow = tmem_base + (uint32_t(quad * 32) << 16);
  if (s_in && hf == 0) {                             // TMEM accesses are warp-wide: every lane stores (rows >= HD: zeros)
#pragma unroll
    for (int c = 0; c < HD / 32; ++c) {
      uint32_t r[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) r[i] = row < HD ? __float_as_uint(s_in[bh * st_stride + (size_t)row * HD + c * 32 + i]) : 0u;
      tmem_st_x32(trow + COL_S + c * 32, r);
    }
    tmem_st_wait();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();

  auto load = [&](uint8_t* dst, const CUtensorMap* tm, uint64_t* bar, int chunk) {
    mbar_expect_tx(bar, L::TILE);
#pragma unroll
    for (int a = 0; a < KA; ++a) tma_load_4d(dst + a * (LA_C * 128), tm, bar, a * 64, h, chunk * LA_C, b);
  };
  const uint32_t k_lbo[2] = {HD == 64 ? uint32_t(2 * L::TILE) : uint32_t(LA_C * 128), HD == 64 ? uint32_t(L::TILE) : uint32_t(LA_C * 128)};
  if (tid == 0) {
    if (full) load(sQ, &tmQ, q_bar, 0);
    load(sK, &tmK, &k_bar[0], 0);
    load(sV, &tmV, v_bar, 0);
    if (n_chunks > 1) load(sK + L::TILE, &tmK, &k_bar[1], 1);
  }
  bool ok = true;
  const bool have_state0 = s_in != nullptr;
  for (int c = 0; c < n_chunks; ++c) {
    const int st = c & 1;
    uint8_t* sKc = sK + st * L::TILE;
    const int valid = min(LA_C, p.S - c * LA_C);
    // ---- phi in place
    if (full && !mbar_wait(q_bar, c & 1, p.status, ST_TIMEOUT_TMA_FULL)) ok = false;
    if (ok && !mbar_wait(&k_bar[st], (c >> 1) & 1, p.status, ST_TIMEOUT_TMA_FULL)) ok = false;
    if (__syncthreads_or(!ok)) { ok = false; break; }
    if (full) la_phi_half<HD>(sQ, row, hf, LA_C, p.scale, p.kind);
    la_phi_half<HD>(sKc, row, hf, valid, p.scale, p.kind);
    fence_proxy_async_smem();
    __syncthreads();
    float den = p.eps;
    if (full) {
      if (tid == 0) {
        tc_fence_after_sync();
        la_mma_xyT<HD>(tmem_base + COL_A, sQ, sKc);                                   // A = Q~ K~^T
        la_mma_pw<HD, HD>(tmem_base + COL_NUM, sQ, sShi, HD * 128, false);            // NUM = Q~ S (value + remainder)
        la_mma_pw<HD, HD>(tmem_base + COL_NUM, sQ, sSlo, HD * 128, true);
        tc_commit(a_bar);                                                             // covers every reader of Q~
      }
      // this half's share of Q~ . z in fp32 while the tensor core works
      float part = la_dot_half<HD>(sQ, row, hf, sz);
      if (!mbar_wait(a_bar, c & 1, p.status, ST_TIMEOUT_ACC_FULL)) ok = false;
      if (__syncthreads_or(!ok)) { ok = false; break; }
      tc_fence_after_sync();
      if (HD == 64 && tid == 0 && c + 1 < n_chunks) load(sQ, &tmQ, q_bar, c + 1);  // Q~ has been consumed
      float a[64];
      la_tmem_row<64>(trow + COL_A + hf * 64, a);
      float r0 = 0.f, r1 = 0.f;
#pragma unroll
      for (int i = 0; i < 64; i += 2) {
        if (hf * 64 + i > row) a[i] = 0.f;
        if (hf * 64 + i + 1 > row) a[i + 1] = 0.f;
        r0 += a[i]; r1 += a[i + 1];
      }
      s_part[hf * LA_C + row] = part + (r0 + r1);
      la_write_half128_hilo(sP, sPlo, row, hf, a, rem);
      tc_fence_before_sync();
      fence_proxy_async_smem();
    }
    __syncthreads();
    if (full) den += s_part[row] + s_part[LA_C + row];        // both halves add in the same order
    if (tid == 0) {
      ok = mbar_wait(v_bar, c & 1, p.status, ST_TIMEOUT_TMA_FULL);
      if (ok) {
        tc_fence_after_sync();
        if (full) {                                                                                    // NUM += A V (value + remainder)
          la_mma_pw<HD, LA_C>(tmem_base + COL_NUM, sP, sV, LA_C * 128, true);
          if (rem) la_mma_pw<HD, LA_C>(tmem_base + COL_NUM, sPlo, sV, LA_C * 128, true);
        }
        la_mma_xTw<HD>(tmem_base + COL_S, sKc, k_lbo[st], sV, have_state0 || c > 0);                   // S += K~^T V
        tc_commit(b_bar);
      }
    }
    // z += colsum(K~) while the products run: ZP row groups per column, combined after the barrier below
    s_zk[tid] = la_colsum_rows(sKc, tid % HD, (tid / HD) * (LA_C / ZP), LA_C / ZP);
    if (!mbar_wait(b_bar, c & 1, p.status, ST_TIMEOUT_ACC_FULL)) ok = false;
    if (__syncthreads_or(!ok)) { ok = false; break; }
    tc_fence_after_sync();
    if (tid == 0) {                                                           // K~ and V of this chunk are free
      if (HD == 128 && full && c + 1 < n_chunks) load(sQ, &tmQ, q_bar, c + 1);  // (its buffer held the remainder tile)
      if (c + 1 < n_chunks) load(sV, &tmV, v_bar, c + 1);
      if (c + 2 < n_chunks) load(sKc, &tmK, &k_bar[st], c + 2);
    }
    if (full) {
      float num[HH];
      la_tmem_row<HH>(trow + COL_NUM + hf * HH, num);
      const int tok = c * LA_C + row;
      if (tok < p.S) {
        const float inv = 1.f / den;
        __nv_bfloat16* op = reinterpret_cast<__nv_bfloat16*>(p.o.ptr) + (long long)b * p.o.sb + (long long)tok * p.o.ss + (long long)h * p.o.sh + hf * HH;
        __nv_bfloat16* lp = p.o_lo.ptr ? reinterpret_cast<__nv_bfloat16*>(p.o_lo.ptr) + (long long)b * p.o_lo.sb + (long long)tok * p.o_lo.ss + (long long)h * p.o_lo.sh + hf * HH : nullptr;
#pragma unroll
        for (int i = 0; i < HH; i += 8) {
          uint32_t hi[4], lo[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float x = num[i + 2 * j] * inv, y = num[i + 2 * j + 1] * inv;
            hi[j] = pack_bf16x2(x, y);
            const float2 r = unpack_bf16x2(hi[j]);
            lo[j] = pack_bf16x2(x - r.x, y - r.y);
          }
          *reinterpret_cast<uint4*>(op + i) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
          if (lp) *reinterpret_cast<uint4*>(lp + i) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
        }
        if (p.den && hf == 0) p.den[((long long)b * p.H + h) * p.S + tok] = den;
      }
    }
    if (tid < HD) {
      float zk = 0.f;
#pragma unroll
      for (int g = 0; g < ZP; ++g) zk += s_zk[g * HD + tid];
      sz[tid] += zk;
    }
    if (full && c + 1 < n_chunks && quad * 32 < HD) {                         // operand copies of the new state (warps that own state rows)
      float srow[HH];
      la_tmem_row<HH>(trow + COL_S + hf * HH, srow);
      if (row < HD) la_write_hilo_half<HD>(sShi, sSlo, HD, row, hf, srow);
      fence_proxy_async_smem();
    }
    tc_fence_before_sync();
    __syncthreads();
  }
  float* s_out = la_publish_begin<HD>(p, bh, sx_epoch, p.s_out);      // the caller's buffer, or this rank's slot of the exchange
  if (ok && s_out && hf == 0) {
    tc_fence_after_sync();
    float srow[HD];
    la_tmem_row<HD>(trow + COL_S, srow);
    if (row < HD) {
#pragma unroll
      for (int i = 0; i < HD; i += 4)
        *reinterpret_cast<float4*>(s_out + bh * st_stride + (size_t)row * HD + i) = make_float4(srow[i], srow[i + 1], srow[i + 2], srow[i + 3]);
      s_out[bh * st_stride + (size_t)HD * HD + row] = sz[row];
    }
  }
  la_publish_end(p, bh, sx_epoch);
  la_retire(p, sx_epoch);
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) { tc_fence_after_sync(); tmem_dealloc(tmem_base, 512); }
}

// dO and O rows of one token -> G = dO / D (bf16 tile row), returns dden = -(dO . O) / D. Tokens past the end give zeros.
template <int HD>
__device__ __forceinline__ float la_load_g(const LinAttnArgs& p, int b, int h, int tok, uint8_t* sG, int row) {
  uint32_t g[HD / 2];
  float dden = 0.f;
  if (tok < p.S) {
    const __nv_bfloat16* dp = reinterpret_cast<const __nv_bfloat16*>(p.dout.ptr) + (long long)b * p.dout.sb + (long long)tok * p.dout.ss + (long long)h * p.dout.sh;
    const __nv_bfloat16* op = reinterpret_cast<const __nv_bfloat16*>(p.o.ptr) + (long long)b * p.o.sb + (long long)tok * p.o.ss + (long long)h * p.o.sh;
    const __nv_bfloat16* lp = p.o_lo.ptr ? reinterpret_cast<const __nv_bfloat16*>(p.o_lo.ptr) + (long long)b * p.o_lo.sb + (long long)tok * p.o_lo.ss + (long long)h * p.o_lo.sh : nullptr;
    const float inv = 1.f / p.den[((long long)b * p.H + h) * p.S + tok];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < HD; i += 8) {
      const uint4 du = *reinterpret_cast<const uint4*>(dp + i), ou = *reinterpret_cast<const uint4*>(op + i);
      const uint4 lu = lp ? *reinterpret_cast<const uint4*>(lp + i) : make_uint4(0, 0, 0, 0);
      const uint32_t* dw = &du.x; const uint32_t* ow = &ou.x; const uint32_t* lw = &lu.x;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 d2 = unpack_bf16x2(dw[j]), o2 = unpack_bf16x2(ow[j]), l2 = unpack_bf16x2(lw[j]);
        // the SAME rounded G enters G V^T on the tensor core and the dot product here, so that the two halves of
        // dA = G . (V_s - O_t) see one dO; O carries its remainder
        const uint32_t gp = pack_bf16x2(d2.x * inv, d2.y * inv);
        const float2 gr = unpack_bf16x2(gp);
        g[(i >> 1) + j] = gp;
        dot = fmaf(gr.x, o2.x + l2.x, dot); dot = fmaf(gr.y, o2.y + l2.y, dot);
      }
    }
    dden = -dot;
  } else {
#pragma unroll
    for (int i = 0; i < HD / 2; ++i) g[i] = 0u;
  }
#pragma unroll
  for (int gi = 0; gi < HD / 8; ++gi)
    *reinterpret_cast<uint4*>(sG + (gi >> 3) * (LA_C * 128) + sw128_offset(row, gi & 7)) =
        make_uint4(g[gi * 4], g[gi * 4 + 1], g[gi * 4 + 2], g[gi * 4 + 3]);
  return dden;
}

// grad[i] <- scale * phi'(scale * x_i) * grad[i] with x the raw (bf16) row in global memory, then store as bf16
template <int HD>
__device__ __forceinline__ void la_store_dphi(const AttnTensor& x, const AttnTensor& dx, int b, int h, int tok, const float* grad, float scale, int kind) {
  const __nv_bfloat16* xp = reinterpret_cast<const __nv_bfloat16*>(x.ptr) + (long long)b * x.sb + (long long)tok * x.ss + (long long)h * x.sh;
  __nv_bfloat16* gp = reinterpret_cast<__nv_bfloat16*>(dx.ptr) + (long long)b * dx.sb + (long long)tok * dx.ss + (long long)h * dx.sh;
#pragma unroll
  for (int i = 0; i < HD; i += 8) {
    const uint4 xu = *reinterpret_cast<const uint4*>(xp + i);
    const uint32_t* xw = &xu.x;
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 x2 = unpack_bf16x2(xw[j]);
      const float a = x2.x * scale, c = x2.y * scale;
      const float da = kind == 0 ? (a > 0.f ? 1.f : __expf(a)) : (a > 0.f ? 2.f * a : 0.f);
      const float dc = kind == 0 ? (c > 0.f ? 1.f : __expf(c)) : (c > 0.f ? 2.f * c : 0.f);
      o[j] = pack_bf16x2(grad[i + 2 * j] * da * scale, grad[i + 2 * j + 1] * dc * scale);
    }
    *reinterpret_cast<uint4*>(gp + i) = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// ---------------------------------------------------------------------------------------------------- backward helpers (8 warps)
// This thread's half of one token: G = dO / D for HD / 2 columns (bf16 tile row), returns its share of -(G . O).
// Tokens past the end give zeros.
template <int HD>
__device__ __forceinline__ float la_load_g_half(const LinAttnArgs& p, int b, int h, int tok, uint8_t* sG, int row, int hf) {
  constexpr int HH = HD / 2;
  uint32_t g[HH / 2];
  float dden = 0.f;
  if (tok < p.S) {
    const __nv_bfloat16* dp = reinterpret_cast<const __nv_bfloat16*>(p.dout.ptr) + (long long)b * p.dout.sb + (long long)tok * p.dout.ss + (long long)h * p.dout.sh + hf * HH;
    const __nv_bfloat16* op = reinterpret_cast<const __nv_bfloat16*>(p.o.ptr) + (long long)b * p.o.sb + (long long)tok * p.o.ss + (long long)h * p.o.sh + hf * HH;
    const __nv_bfloat16* lp = p.o_lo.ptr ? reinterpret_cast<const __nv_bfloat16*>(p.o_lo.ptr) + (long long)b * p.o_lo.sb + (long long)tok * p.o_lo.ss + (long long)h * p.o_lo.sh + hf * HH : nullptr;
    const float inv = 1.f / p.den[((long long)b * p.H + h) * p.S + tok];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < HH; i += 8) {
      const uint4 du = *reinterpret_cast<const uint4*>(dp + i), ou = *reinterpret_cast<const uint4*>(op + i);
      const uint4 lu = lp ? *reinterpret_cast<const uint4*>(lp + i) : make_uint4(0, 0, 0, 0);
      const uint32_t* dw = &du.x; const uint32_t* ow = &ou.x; const uint32_t* lw = &lu.x;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 d2 = unpack_bf16x2(dw[j]), o2 = unpack_bf16x2(ow[j]), l2 = unpack_bf16x2(lw[j]);
        // the SAME rounded G enters G V^T on the tensor core and the dot product here; O carries its remainder
        const uint32_t gp = pack_bf16x2(d2.x * inv, d2.y * inv);
        const float2 gr = unpack_bf16x2(gp);
        g[(i >> 1) + j] = gp;
        dot = fmaf(gr.x, o2.x + l2.x, dot); dot = fmaf(gr.y, o2.y + l2.y, dot);
      }
    }
    dden = -dot;
  } else {
#pragma unroll
    for (int i = 0; i < HH / 2; ++i) g[i] = 0u;
  }
#pragma unroll
  for (int gi = 0; gi < HH / 8; ++gi) {
    const int gc = hf * (HH / 8) + gi;                 // 16-byte chunk of the full row
    *reinterpret_cast<uint4*>(sG + (gc >> 3) * (LA_C * 128) + sw128_offset(row, gc & 7)) =
        make_uint4(g[gi * 4], g[gi * 4 + 1], g[gi * 4 + 2], g[gi * 4 + 3]);
  }
  return dden;
}
// grad[i] <- scale * phi'(scale * x_i) * grad[i] for this thread's HD / 2 columns of a token, stored as bf16
template <int HD>
__device__ __forceinline__ void la_store_dphi_half(const AttnTensor& x, const AttnTensor& dx, int b, int h, int tok, int hf, const float* grad, float scale, int kind) {
  constexpr int HH = HD / 2;
  const __nv_bfloat16* xp = reinterpret_cast<const __nv_bfloat16*>(x.ptr) + (long long)b * x.sb + (long long)tok * x.ss + (long long)h * x.sh + hf * HH;
  __nv_bfloat16* gp = reinterpret_cast<__nv_bfloat16*>(dx.ptr) + (long long)b * dx.sb + (long long)tok * dx.ss + (long long)h * dx.sh + hf * HH;
#pragma unroll
  for (int i = 0; i < HH; i += 8) {
    const uint4 xu = *reinterpret_cast<const uint4*>(xp + i);
    const uint32_t* xw = &xu.x;
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 x2 = unpack_bf16x2(xw[j]);
      const float a = x2.x * scale, c = x2.y * scale;
      const float da = kind == 0 ? (a > 0.f ? 1.f : __expf(a)) : (a > 0.f ? 2.f * a : 0.f);
      const float dc = kind == 0 ? (c > 0.f ? 1.f : __expf(c)) : (c > 0.f ? 2.f * c : 0.f);
      o[j] = pack_bf16x2(grad[i + 2 * j] * da * scale, grad[i + 2 * j + 1] * dc * scale);
    }
    *reinterpret_cast<uint4*>(gp + i) = make_uint4(o[0], o[1], o[2], o[3]);
  }
}
// partial weighted column sum: sum over rows [r0, r0 + n) of w[r] * tile(r, k)
__device__ __forceinline__ float la_colsum_w_rows(const uint8_t* tile, int k, const float* w, int r0, int n) {
  const uint8_t* base = tile + (k >> 6) * (LA_C * 128) + (k & 7) * 2;
  const int chunk = (k & 63) >> 3;
  float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll 4
  for (int r = r0; r < r0 + n; r += 4) {
    s0 = fmaf(w[r], __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(base + sw128_offset(r, chunk))), s0);
    s1 = fmaf(w[r + 1], __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(base + sw128_offset(r + 1, chunk))), s1);
    s2 = fmaf(w[r + 2], __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(base + sw128_offset(r + 2, chunk))), s2);
    s3 = fmaf(w[r + 3], __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(base + sw128_offset(r + 3, chunk))), s3);
  }
  return (s0 + s1) + (s2 + s3);
}

// ---------------------------------------------------------------------------------------------------- backward 1: dQ
// Same 8-warp mapping as the forward: warp w owns rows 32 (w & 3) .. and column half w >> 2.
template <int HD>
__global__ void __launch_bounds__(LA_FWD_THREADS, 1)
linattn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV, const LinAttnArgs p) {
  using L = LaSmem<HD>;
  constexpr int KA = HD / 64;
  constexpr int HH = HD / 2;
  constexpr int ZP = LA_FWD_THREADS / HD;
  constexpr uint32_t COL_A = 0, COL_DQ = 128, COL_S = 256;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* sG = smem;
  uint8_t* sK = sG + L::TILE;                 // 2 stages
  uint8_t* sZero = sK + 2 * L::TILE;
  uint8_t* sV = sZero + L::ZERO;
  uint8_t* sP = sV + L::TILE;
  uint8_t* sShi = sP + L::PT;
  uint8_t* sSlo = sShi + L::ST;
  uint8_t* sPlo = HD == 64 ? sSlo + L::ST : sG;
  float* sz = reinterpret_cast<float*>(sSlo + L::ST + L::PLO);
  float* s_part = sz + HD;                    // [2][128]: the halves' shares of dden; later in the chunk: partial column sums
  float* s_zk = s_part;                       // (two barriers lie between the last read of one use and the first write of the other)
  float* s_dden = s_part + 2 * LA_C;          // [128]
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_dden + LA_C);
  uint64_t* k_bar = bars; uint64_t* v_bar = bars + 2; uint64_t* a_bar = bars + 3; uint64_t* b_bar = bars + 4;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 5);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int quad = warp & 3, hf = warp >> 2, row = quad * 32 + lane;
  const int bh = blockIdx.x, b = bh / p.H, h = bh % p.H;
  const int n_chunks = (p.S + LA_C - 1) / LA_C;
  const bool rem = p.kind == 0;                // see the forward kernel
  if ((smem_u32(smem) & 1023u) != 0) { if (tid == 0 && p.status) atomicCAS(p.status, 0u, (uint32_t)ST_BAD_ARGUMENT); return; }
  if (tid == 0) {
    mbar_init(&k_bar[0], 1); mbar_init(&k_bar[1], 1); mbar_init(v_bar, 1); mbar_init(a_bar, 1); mbar_init(b_bar, 1);
    fence_barrier_init();
    tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
  }
  if (warp == 0) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  if (HD == 64) for (int i = tid; i < L::ZERO / 16; i += LA_FWD_THREADS) reinterpret_cast<uint4*>(sZero)[i] = make_uint4(0, 0, 0, 0);
  const size_t st_stride = (size_t)HD * HD + HD;
  if (tid < HD) {
    float s0[HD];
#pragma unroll
    for (int i = 0; i < HD; ++i) s0[i] = p.s_in ? p.s_in[bh * st_stride + (size_t)tid * HD + i] : 0.f;
    la_write_hilo<HD>(sShi, sSlo, HD, tid, s0);
    sz[tid] = p.s_in ? p.s_in[bh * st_stride + (size_t)HD * HD + tid] : 0.f;
  }
  tc_fence_before_sync();
  fence_proxy_async_smem();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t trow = tmem_base + (uint32_t(quad * 32) << 16);
  if (p.s_in && hf == 0) {
#pragma unroll
    for (int c = 0; c < HD / 32; ++c) {
      uint32_t r[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) r[i] = row < HD ? __float_as_uint(p.s_in[bh * st_stride + (size_t)row * HD + c * 32 + i]) : 0u;
      tmem_st_x32(trow + COL_S + c * 32, r);
    }
    tmem_st_wait();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();

  auto load = [&](uint8_t* dst, const CUtensorMap* tm, uint64_t* bar, int chunk) {
    mbar_expect_tx(bar, L::TILE);
#pragma unroll
    for (int a = 0; a < KA; ++a) tma_load_4d(dst + a * (LA_C * 128), tm, bar, a * 64, h, chunk * LA_C, b);
  };
  const uint32_t k_lbo[2] = {HD == 64 ? uint32_t(2 * L::TILE) : uint32_t(LA_C * 128), HD == 64 ? uint32_t(L::TILE) : uint32_t(LA_C * 128)};
  if (tid == 0) {
    load(sK, &tmK, &k_bar[0], 0);
    load(sV, &tmV, v_bar, 0);
    if (n_chunks > 1) load(sK + L::TILE, &tmK, &k_bar[1], 1);
  }
  bool ok = true;
  const bool have_state0 = p.s_in != nullptr;
  for (int c = 0; c < n_chunks; ++c) {
    const int st = c & 1;
    uint8_t* sKc = sK + st * L::TILE;
    const int valid = min(LA_C, p.S - c * LA_C);
    const int tok = c * LA_C + row;
    // this half of G and its share of dden come straight from global memory while the TMA tiles land
    s_part[hf * LA_C + row] = la_load_g_half<HD>(p, b, h, tok, sG, row, hf);
    if (!mbar_wait(&k_bar[st], (c >> 1) & 1, p.status, ST_TIMEOUT_TMA_FULL)) ok = false;
    if (ok && !mbar_wait(v_bar, c & 1, p.status, ST_TIMEOUT_TMA_FULL)) ok = false;
    if (__syncthreads_or(!ok)) { ok = false; break; }
    const float dden = s_part[row] + s_part[LA_C + row];
    la_phi_half<HD>(sKc, row, hf, valid, p.scale, p.kind);
    fence_proxy_async_smem();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after_sync();
      la_mma_xyT<HD>(tmem_base + COL_A, sG, sV);                                      // T = G V^T
      la_mma_xwT<HD>(tmem_base + COL_DQ, sG, sShi, false);                            // dQ~ = G S^T (value + remainder)
      la_mma_xwT<HD>(tmem_base + COL_DQ, sG, sSlo, true);
      tc_commit(a_bar);
    }
    if (!mbar_wait(a_bar, c & 1, p.status, ST_TIMEOUT_ACC_FULL)) ok = false;
    if (__syncthreads_or(!ok)) { ok = false; break; }
    tc_fence_after_sync();
    {
      float a[64];
      la_tmem_row<64>(trow + COL_A + hf * 64, a);
#pragma unroll
      for (int i = 0; i < 64; ++i) a[i] = (hf * 64 + i > row) ? 0.f : a[i] + dden;
      la_write_half128_hilo(sP, sPlo, row, hf, a, rem);
    }
    tc_fence_before_sync();
    fence_proxy_async_smem();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after_sync();
      la_mma_pw<HD, LA_C>(tmem_base + COL_DQ, sP, sKc, LA_C * 128, true);             // dQ~ += dA K~ (value + remainder)
      if (rem) la_mma_pw<HD, LA_C>(tmem_base + COL_DQ, sPlo, sKc, LA_C * 128, true);
      la_mma_xTw<HD>(tmem_base + COL_S, sKc, k_lbo[st], sV, have_state0 || c > 0);    // S += K~^T V
      tc_commit(b_bar);
    }
    s_zk[tid] = la_colsum_rows(sKc, tid % HD, (tid / HD) * (LA_C / ZP), LA_C / ZP);
    if (!mbar_wait(b_bar, c & 1, p.status, ST_TIMEOUT_ACC_FULL)) ok = false;
    if (__syncthreads_or(!ok)) { ok = false; break; }
    tc_fence_after_sync();
    if (tid == 0) {
      if (c + 1 < n_chunks) load(sV, &tmV, v_bar, c + 1);
      if (c + 2 < n_chunks) load(sKc, &tmK, &k_bar[st], c + 2);
    }
    {
      float dq[HH];
      la_tmem_row<HH>(trow + COL_DQ + hf * HH, dq);
      if (tok < p.S) {
#pragma unroll
        for (int i = 0; i < HH; ++i) dq[i] = fmaf(dden, sz[hf * HH + i], dq[i]);      // z of the chunks before this one
        la_store_dphi_half<HD>(p.q, p.dq, b, h, tok, hf, dq, p.scale, p.kind);
      }
    }
    __syncthreads();                                                                  // every thread has read the old z
    if (tid < HD) {
      float zk = 0.f;
#pragma unroll
      for (int g = 0; g < ZP; ++g) zk += s_zk[g * HD + tid];
      sz[tid] += zk;
    }
    if (c + 1 < n_chunks && quad * 32 < HD) {
      float srow[HH];
      la_tmem_row<HH>(trow + COL_S + hf * HH, srow);
      if (row < HD) la_write_hilo_half<HD>(sShi, sSlo, HD, row, hf, srow);
      fence_proxy_async_smem();
    }
    tc_fence_before_sync();
    __syncthreads();
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) { tc_fence_after_sync(); tmem_dealloc(tmem_base, 512); }
}

// ---------------------------------------------------------------------------------------------------- backward 2: dK, dV
template <int HD>
__global__ void __launch_bounds__(LA_FWD_THREADS, 1)
linattn_bwd_dkv_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                       const __grid_constant__ CUtensorMap tmV, const LinAttnArgs p) {
  using L = LaSmem<HD>;
  constexpr int KA = HD / 64;
  constexpr int HH = HD / 2;
  constexpr int ZP = LA_FWD_THREADS / HD;
  constexpr uint32_t COL_T = 0, COL_DV = 128, COL_DK = 128 + HD, COL_DS = 128 + 2 * HD;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* sQ = smem;
  uint8_t* sZero = sQ + L::TILE;               // HD = 64: pads Q~^T G to 128 rows
  uint8_t* sK = sZero + L::ZERO;
  uint8_t* sV = sK + L::TILE;
  uint8_t* sG = sV + L::TILE;
  uint8_t* sP = sG + L::TILE;
  uint8_t* sDhi = sP + L::PT;
  uint8_t* sDlo = sDhi + L::ST;
  float* sdz = reinterpret_cast<float*>(sDlo + L::ST);     // [HD]
  float* sdden = sdz + HD;                                  // [128]
  float* s_part = sdden + LA_C;                             // [2][128] dden shares; later in the chunk: partial column sums
  float* s_zk = s_part;
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_part + 2 * LA_C);
  uint64_t* ld_bar = bars; uint64_t* t_bar = bars + 1; uint64_t* u_bar = bars + 2; uint64_t* b_bar = bars + 3;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 4);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int quad = warp & 3, hf = warp >> 2, row = quad * 32 + lane;
  const int bh = blockIdx.x, b = bh / p.H, h = bh % p.H;
  const int n_chunks = (p.S + LA_C - 1) / LA_C;
  const bool full = !p.state_only;               // state_only: only dS / dz of this slice (reads Q, dO, O)
  if ((smem_u32(smem) & 1023u) != 0) { if (tid == 0 && p.status) atomicCAS(p.status, 0u, (uint32_t)ST_BAD_ARGUMENT); return; }
  if (tid == 0) {
    mbar_init(ld_bar, 1); mbar_init(t_bar, 1); mbar_init(u_bar, 1); mbar_init(b_bar, 1);
    fence_barrier_init();
    tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
  }
  if (warp == 0) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  if (HD == 64) for (int i = tid; i < L::ZERO / 16; i += LA_FWD_THREADS) reinterpret_cast<uint4*>(sZero)[i] = make_uint4(0, 0, 0, 0);
  const size_t st_stride = (size_t)HD * HD + HD;
  const uint32_t sx_epoch = la_epoch(p);
  const float* ds_in = la_consume<HD>(p, bh, sx_epoch, p.ds_in);     // the caller's dS, or the higher ranks' totals
  if (tid < HD) {
    float s0[HD];
#pragma unroll
    for (int i = 0; i < HD; ++i) s0[i] = ds_in ? ds_in[bh * st_stride + (size_t)tid * HD + i] : 0.f;
    la_write_hilo<HD>(sDhi, sDlo, HD, tid, s0);
    sdz[tid] = ds_in ? ds_in[bh * st_stride + (size_t)HD * HD + tid] : 0.f;
  }
  tc_fence_before_sync();
  fence_proxy_async_smem();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t trow = tmem_base + (uint32_t(quad * 32) << 16);
  if (ds_in && hf == 0) {
#pragma unroll
    for (int c = 0; c < HD / 32; ++c) {
      uint32_t r[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) r[i] = row < HD ? __float_as_uint(ds_in[bh * st_stride + (size_t)row * HD + c * 32 + i]) : 0u;
      tmem_st_x32(trow + COL_DS + c * 32, r);
    }
    tmem_st_wait();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();

  auto load_all = [&](int chunk) {                      // Q, K, V tiles of one chunk on one barrier
    mbar_expect_tx(ld_bar, 3 * L::TILE);
#pragma unroll
    for (int a = 0; a < KA; ++a) {
      tma_load_4d(sQ + a * (LA_C * 128), &tmQ, ld_bar, a * 64, h, chunk * LA_C, b);
      tma_load_4d(sK + a * (LA_C * 128), &tmK, ld_bar, a * 64, h, chunk * LA_C, b);
      tma_load_4d(sV + a * (LA_C * 128), &tmV, ld_bar, a * 64, h, chunk * LA_C, b);
    }
  };
  const uint32_t q_lbo = HD == 64 ? uint32_t(L::TILE) : uint32_t(LA_C * 128);
  if (tid == 0) load_all(n_chunks - 1);
  bool ok = true;
  const bool have_state0 = ds_in != nullptr;
  uint32_t t_phase = 0;
  for (int it = 0; it < n_chunks; ++it) {
    const int c = n_chunks - 1 - it;
    const int valid = min(LA_C, p.S - c * LA_C);
    const int tok = c * LA_C + row;
    s_part[hf * LA_C + row] = la_load_g_half<HD>(p, b, h, tok, sG, row, hf);
    if (!mbar_wait(ld_bar, it & 1, p.status, ST_TIMEOUT_TMA_FULL)) ok = false;
    if (__syncthreads_or(!ok)) { ok = false; break; }
    if (hf == 0) sdden[row] = s_part[row] + s_part[LA_C + row];
    la_phi_half<HD>(sQ, row, hf, LA_C, p.scale, p.kind);
    if (full) la_phi_half<HD>(sK, row, hf, valid, p.scale, p.kind);
    fence_proxy_async_smem();
    __syncthreads();
    if (full) {
    if (tid == 0) {
      tc_fence_after_sync();
      la_mma_xyT<HD>(tmem_base + COL_T, sK, sQ);                                      // A^T = K~ Q~^T   [key][query]
      tc_commit(t_bar);
      la_mma_pw<HD, HD>(tmem_base + COL_DV, sK, sDhi, HD * 128, false);               // dV = K~ dS (value + remainder)
      la_mma_pw<HD, HD>(tmem_base + COL_DV, sK, sDlo, HD * 128, true);
      la_mma_xwT<HD>(tmem_base + COL_DK, sV, sDhi, false);                            // dK~ = V dS^T
      la_mma_xwT<HD>(tmem_base + COL_DK, sV, sDlo, true);
    }
    if (!mbar_wait(t_bar, t_phase, p.status, ST_TIMEOUT_ACC_FULL)) ok = false;
    t_phase ^= 1;
    if (__syncthreads_or(!ok)) { ok = false; break; }
    tc_fence_after_sync();
    {
      float a[64];
      la_tmem_row<64>(trow + COL_T + hf * 64, a);
#pragma unroll
      for (int i = 0; i < 64; ++i) if (hf * 64 + i < row) a[i] = 0.f;                // keep queries at or after this key
      la_write_half128_hilo(sP, sP, row, hf, a, false);
    }
    tc_fence_before_sync();
    fence_proxy_async_smem();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after_sync();
      la_mma_pw<HD, LA_C>(tmem_base + COL_DV, sP, sG, LA_C * 128, true);              // dV += mask(A)^T G
      tc_commit(u_bar);
      la_mma_xyT<HD>(tmem_base + COL_T, sV, sG);                                      // (G V^T)^T = V G^T   [key][query]
      tc_commit(t_bar);
    }
    if (!mbar_wait(t_bar, t_phase, p.status, ST_TIMEOUT_ACC_FULL)) ok = false;      // implies u_bar: the tensor core runs in order
    t_phase ^= 1;
    if (ok && !mbar_wait(u_bar, it & 1, p.status, ST_TIMEOUT_ACC_FULL)) ok = false;
    if (__syncthreads_or(!ok)) { ok = false; break; }
    tc_fence_after_sync();
    {
      float a[64];
      la_tmem_row<64>(trow + COL_T + hf * 64, a);
#pragma unroll
      for (int i = 0; i < 64; ++i) a[i] = (hf * 64 + i < row) ? 0.f : a[i] + sdden[hf * 64 + i];
      la_write_half128_hilo(sP, sP, row, hf, a, false);
    }
    tc_fence_before_sync();
    fence_proxy_async_smem();
    }
    __syncthreads();
    if (tid == 0) {
      tc_fence_after_sync();
      if (full) la_mma_pw<HD, LA_C>(tmem_base + COL_DK, sP, sQ, LA_C * 128, true);    // dK~ += mask(dA)^T Q~
      la_mma_xTw<HD>(tmem_base + COL_DS, sQ, q_lbo, sG, have_state0 || it > 0);       // dS += Q~^T G
      tc_commit(b_bar);
    }
    // dz += Q~^T dden in fp32: ZP row groups per column, combined after the barriers below
    s_zk[tid] = la_colsum_w_rows(sQ, tid % HD, sdden, (tid / HD) * (LA_C / ZP), LA_C / ZP);
    if (!mbar_wait(b_bar, it & 1, p.status, ST_TIMEOUT_ACC_FULL)) ok = false;
    if (__syncthreads_or(!ok)) { ok = false; break; }
    tc_fence_after_sync();
    if (tid == 0 && c > 0) load_all(c - 1);
    if (full) {
      float g[HH];
      la_tmem_row<HH>(trow + COL_DV + hf * HH, g);
      if (tok < p.S) {
        __nv_bfloat16* vp = reinterpret_cast<__nv_bfloat16*>(p.dv.ptr) + (long long)b * p.dv.sb + (long long)tok * p.dv.ss + (long long)h * p.dv.sh + hf * HH;
#pragma unroll
        for (int i = 0; i < HH; i += 8)
          *reinterpret_cast<uint4*>(vp + i) = make_uint4(pack_bf16x2(g[i], g[i + 1]), pack_bf16x2(g[i + 2], g[i + 3]),
                                                         pack_bf16x2(g[i + 4], g[i + 5]), pack_bf16x2(g[i + 6], g[i + 7]));
      }
      la_tmem_row<HH>(trow + COL_DK + hf * HH, g);
      if (tok < p.S) {
#pragma unroll
        for (int i = 0; i < HH; ++i) g[i] += sdz[hf * HH + i];                         // dz of the chunks after this one
        la_store_dphi_half<HD>(p.k, p.dk, b, h, tok, hf, g, p.scale, p.kind);
      }
    }
    __syncthreads();                                                                  // every thread has read the old dz
    if (tid < HD) {
      float dzk = 0.f;
#pragma unroll
      for (int g = 0; g < ZP; ++g) dzk += s_zk[g * HD + tid];
      sdz[tid] += dzk;
    }
    if (full && c > 0 && quad * 32 < HD) {
      float srow[HH];
      la_tmem_row<HH>(trow + COL_DS + hf * HH, srow);
      if (row < HD) la_write_hilo_half<HD>(sDhi, sDlo, HD, row, hf, srow);
      fence_proxy_async_smem();
    }
    tc_fence_before_sync();
    __syncthreads();
  }
  float* ds_out = la_publish_begin<HD>(p, bh, sx_epoch, p.ds_out);
  if (ok && ds_out && hf == 0) {
    tc_fence_after_sync();
    float srow[HD];
    la_tmem_row<HD>(trow + COL_DS, srow);
    if (row < HD) {
#pragma unroll
      for (int i = 0; i < HD; i += 4)
        *reinterpret_cast<float4*>(ds_out + bh * st_stride + (size_t)row * HD + i) = make_float4(srow[i], srow[i + 1], srow[i + 2], srow[i + 3]);
      ds_out[bh * st_stride + (size_t)HD * HD + row] = sdz[row];
    }
  }
  la_publish_end(p, bh, sx_epoch);
  la_retire(p, sx_epoch);
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) { tc_fence_after_sync(); tmem_dealloc(tmem_base, 512); }
}

// ---------------------------------------------------------------------------------------------------- host side
template <int HD> constexpr int la_fwd_smem() { return 4 * LaSmem<HD>::TILE + LaSmem<HD>::ZERO + LaSmem<HD>::PT + LaSmem<HD>::PLO + 2 * LaSmem<HD>::ST + HD * 4 + 128; }
// the forward kernel also keeps [2][128] denominator shares and 256 partial column sums
template <int HD> constexpr int la_fwd8_smem() { return la_fwd_smem<HD>() + 2 * LA_C * 4 + LA_FWD_THREADS * 4; }
// dQ: [2][128] dden shares (reused for the partial column sums) + [128] dden; dK / dV: the same shares beside its [128] dden
template <int HD> constexpr int la_dq8_smem() { return la_fwd_smem<HD>() + 3 * LA_C * 4; }
template <int HD> constexpr int la_dkv_smem() { return 4 * LaSmem<HD>::TILE + LaSmem<HD>::ZERO + LaSmem<HD>::PT + 2 * LaSmem<HD>::ST + (HD + LA_C) * 4 + 2 * LA_C * 4 + 128; }

static int la_maps(const LinAttnArgs& a, CUtensorMap* tq, CUtensorMap* tk, CUtensorMap* tv) {
  const auto BF = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  if (tq && make_tmap_attn(tq, a.q.ptr, BF, 2, a.hd, a.H, a.S, a.B, a.q.sh, a.q.ss, a.q.sb, 64, LA_C, CU_TENSOR_MAP_SWIZZLE_128B)) return 101;
  if (make_tmap_attn(tk, a.k.ptr, BF, 2, a.hd, a.H, a.S, a.B, a.k.sh, a.k.ss, a.k.sb, 64, LA_C, CU_TENSOR_MAP_SWIZZLE_128B)) return 102;
  if (make_tmap_attn(tv, a.v.ptr, BF, 2, a.hd, a.H, a.S, a.B, a.v.sh, a.v.ss, a.v.sb, 64, LA_C, CU_TENSOR_MAP_SWIZZLE_128B)) return 103;
  return 0;
}

template <int HD>
static int la_set_attrs() {
  static bool done = false;
  if (done) return 0;
  (void)cudaGetLastError();
  if (cudaFuncSetAttribute(linattn_fwd_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, la_fwd8_smem<HD>()) != cudaSuccess) return 1;
  if (cudaFuncSetAttribute(linattn_bwd_dq_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, la_dq8_smem<HD>()) != cudaSuccess) return 1;
  if (cudaFuncSetAttribute(linattn_bwd_dkv_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, la_dkv_smem<HD>()) != cudaSuccess) return 1;
  done = true;
  return 0;
}

template <int HD>
static int la_launch(const LinAttnArgs& a, int which, cudaStream_t st) {
  if (la_set_attrs<HD>()) return 104;
  CUtensorMap tq, tk, tv;
  const bool need_q = which != 1 && !(which == 0 && a.state_only);
  if (int rc = la_maps(a, need_q ? &tq : nullptr, &tk, &tv)) return rc;
  if (!need_q) tq = tk;
  const unsigned grid = (unsigned)(a.B * a.H);
  if (which == 0) linattn_fwd_kernel<HD><<<grid, LA_FWD_THREADS, la_fwd8_smem<HD>(), st>>>(tq, tk, tv, a);
  else if (which == 1) linattn_bwd_dq_kernel<HD><<<grid, LA_FWD_THREADS, la_dq8_smem<HD>(), st>>>(tk, tv, a);
  else linattn_bwd_dkv_kernel<HD><<<grid, LA_FWD_THREADS, la_dkv_smem<HD>(), st>>>(tq, tk, tv, a);
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}

}  // namespace b200

// which: 0 forward (or state-only pass), 1 backward dQ, 2 backward dK / dV. Causal form; hd 64 or 128; bf16.
extern "C" int b200_linattn(const b200::LinAttnArgs* a, int which, cudaStream_t st) {
  using namespace b200;
  if (a->B <= 0 || a->H <= 0 || a->S <= 0) return 0;
  if (which < 0 || which > 2) return -2;
  if (a->hd == 64) return la_launch<64>(*a, which, st);
  if (a->hd == 128) return la_launch<128>(*a, which, st);
  return -3;
}
extern "C" int b200_linattn_init() { return b200::la_set_attrs<64>() | b200::la_set_attrs<128>(); }
