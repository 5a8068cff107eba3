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
