// Launch interface of the tcgen05 GEMM family (plain C structs; no torch dependency).
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace b200 {

enum : int { ACT_NONE = 0, ACT_RELU = 1, ACT_GELU = 2, ACT_SILU = 3, ACT_SIGMOID = 4, ACT_TANH = 5 };
enum : int { OUT_BF16 = 0, OUT_F32 = 1, OUT_F32_ATOMIC = 2, OUT_I32 = 3 };   // OUT_I32: raw int32 accumulators (int8 kinds only)
enum : int { GEMM_BF16 = 0, GEMM_F32 = 1, GEMM_S8S8 = 2, GEMM_U8S8 = 3, GEMM_E4M3 = 4 };

// Device-visible parameters. Strides are in elements of the respective tensor.
struct GemmParams {
  int M, N, K, batch;
  int splits;              // split-K factor; >1 requires OUT_F32_ATOMIC
  void* C; long long ldc, strideC;
  const void* bias; int bias_f32; int bias_vec_ok;   // bias_vec_ok: fp32 bias is 16-byte aligned
  long long strideBias;    // elements between the bias vectors of consecutive batches (0: shared)
  const void* residual; long long ldr, strideR;   // bf16, added after the activation
  void* aux_out;           // bf16 copy of the pre-activation value (layout of C)
  const void* aux_in;      // bf16 saved value; result is multiplied by act'(aux_in) (layout of C)
  float alpha;
  const float* alpha_ptr;   // optional device scalar multiplied into alpha (e.g. an upstream loss gradient)
  int act, dact, out_mode;
  int vec_ok, res_vec_ok;  // 16-byte vector access is legal for C/aux and for residual
  const float* row_scale;  // 8-bit kinds: fp32 dequantisation scale per row of A ([batch*M]) or null
  const float* col_scale;  // 8-bit kinds: fp32 dequantisation scale per column (row of B, [N]) or null
  uint32_t* status;        // device word, receives a non-zero code on a bounded-wait expiry
  // Grouped (batched) products over ragged groups, e.g. the tokens routed to each expert: device arrays [batch] or null.
  const int* m_valid;      // rows of A (and C) in use per batch: row tiles wholly past it are skipped (their C rows are not written)
  const int* k_valid;      // contraction length in use per batch, rounded up to 128: the K loop stops there
};

// Tensor-parallel extension: the GEMM fused with the collective next to it, over NVLink peer memory.
//   TP_AG_GEMM (all-gather -> GEMM): A's row blocks belong to `world` ranks. A few CTAs of the grid push
//     this rank's rows into every peer's staging copy of A (one NVLink crossing per element and peer) and
//     release a per-row-block flag at the peer; the TMA producers of the GEMM CTAs wait on their local
//     flags, so tiles of rows that have arrived multiply while later rows are still in flight.
//   TP_GEMM_RS (GEMM -> reduce-scatter): every rank holds a K-slice and computes a partial C. The
//     epilogue stores each row block straight into its owner's slot buffer (plain 16-byte peer stores),
//     the last CTA runs a cross-rank handshake, then all CTAs sum the `world` slots of the local rows
//     (+ residual) into the output.
enum : int { TP_NONE = 0, TP_AG_GEMM = 1, TP_GEMM_RS = 2 };
constexpr int TP_MAX_WORLD = 8;
struct TpParams {
  int mode, rank, world, copy_ctas;
  int blocks_per_rank;               // row blocks of 128 rows per rank (M / world / 128)
  uint32_t* epoch_ptr;               // local device word: calls so far on this context; the call uses *epoch_ptr + 1 and stores it back
  long long wait_cycles;             // clock64 budget of one wait
  // TP_AG_GEMM
  void* stage_peer[TP_MAX_WORLD];    // every rank's staging buffer [M, K] bf16 (peer-mapped); rank r fills rows r*M/world.. of
                                     // its own copy before the call, the gather CTAs push them into all the others
  uint32_t* ready_peer[TP_MAX_WORLD];// every rank's per-row-block flags (peer-mapped): written by the pushing rank
  // TP_GEMM_RS
  void* slots_peer[TP_MAX_WORLD];    // every rank's slot buffer [2][world][rows_per_rank][N] bf16 (peer-mapped)
  void* out;                         // local result [rows_per_rank, N] bf16
  uint32_t* go;                      // local word: "all peers' partials have landed"
  // both
  uint32_t* flags[TP_MAX_WORLD];     // every rank's flag words [2][TP_MAX_WORLD] (peer-mapped): [0] shard ready, [1] done
  uint32_t* done_ctr;                // local counter of finished CTAs
};

struct GemmArgs {
  GemmParams p;
  const void* A; long long lda, strideA; int a_mn;   // a_mn: A stored [K,M] (M contiguous)
  const void* B; long long ldb, strideB; int b_mn;   // b_mn: B stored [K,N] (N contiguous)
  int M, N, K, batch;
  int dtype;               // GEMM_BF16 / GEMM_F32 (runs as TF32) / GEMM_S8S8 / GEMM_U8S8 / GEMM_E4M3
};

}  // namespace b200

extern "C" int b200_gemm_launch(const b200::GemmArgs* args, int bn, int num_sms, cudaStream_t stream);
extern "C" int b200_gemm_tp_launch(const b200::GemmArgs* args, const b200::TpParams* tp, int bn, int num_sms, cudaStream_t stream);
