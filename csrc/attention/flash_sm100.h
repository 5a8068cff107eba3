// Launch interface of the tcgen05 FlashAttention kernels (A1 forward, A2 backward).
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace b200 {

// Element (b, s, h, e) of a tensor lives at ptr + b*sb + s*ss + h*sh + e (strides in elements).
struct AttnTensor { void* ptr; long long sb, ss, sh; };

struct FlashArgs {
  AttnTensor q, k, v, o;        // bf16
  AttnTensor dout, dq, dk, dv;  // bf16 (backward only)
  float* lse;                   // [B, H, Sq] fp32, natural-log log-sum-exp of the scaled scores
  float* delta;                 // [B, H, Sq] fp32 scratch: rowsum(dO * O) (backward only)
  float* dq_accum;              // [B, Sq, H, hd] fp32 scratch, zeroed by the launcher (backward only)
  int B, H, Sq, Skv, hd;
  float scale;
  int causal;
  uint32_t* status;
};

}  // namespace b200

extern "C" int b200_flash_fwd(const b200::FlashArgs* a, cudaStream_t st);
extern "C" int b200_flash_bwd(const b200::FlashArgs* a, cudaStream_t st);
