// A5: exchange of linear-attention KV states between sequence-parallel ranks.
//
// With the sequence split over `world` ranks, causal linear attention needs, on rank r, the sum of
// the [d x (d_v+1)] states of all tokens owned by ranks < r (its backward needs the sum of the state
// gradients of ranks > r; the non-causal form needs the sum over every rank). The states are tiny
// compared with the activations (B*H*d*(d+8) floats), so instead of a ring or an all-gather each rank
// publishes its total once in peer-mapped memory and reads exactly the peers it needs:
//   1. copy the local total into this rank's slot (symmetric memory)
//   2. per-CTA flag handshake with every peer (bounded wait; expiry -> status word, kernel returns)
//   3. sum the selected peers' slots with plain peer loads (no multimem: safe when a rank has left)
//   4. second handshake: nobody's slot is overwritten by the next call while a peer still reads it
// The reference has no sequence parallelism; its O(N) state recurrence is src/linear_attention.rs:110-300.
#include <cuda_runtime.h>
#include <cstdint>
#include "../common/ptx.cuh"

namespace b200 {

constexpr int SX_MAX_WORLD = 8;
constexpr int SX_MAX_CTAS = 64;

struct StateExchangeArgs {
  float* slot[SX_MAX_WORLD];        // every rank's slot [numel] fp32 (peer-mapped)
  uint32_t* flags[SX_MAX_WORLD];    // every rank's flag words [2][SX_MAX_WORLD][SX_MAX_CTAS] (peer-mapped)
  const float* inp;                 // local total state [numel]
  float* out;                       // local result [numel]
  long long numel;                  // multiple of 4
  int rank, world;
  int mode;                         // 0: sum of ranks < rank, 1: sum of ranks > rank, 2: sum of all ranks
  uint32_t epoch;                   // used when `words` is null (a caller that numbers its calls itself)
  long long wait_cycles;
  uint32_t* status;
  uint32_t* words;                  // local device words: [0] calls so far (this call's epoch is [0] + 1; the last CTA to
                                    // retire stores it back, so a replayed launch gets a fresh epoch), [1] retired CTAs
};

__device__ __forceinline__ void sx_st_release(uint32_t* p, uint32_t v) { asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
__device__ __forceinline__ uint32_t sx_ld_acquire(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ bool sx_handshake(const StateExchangeArgs& a, int phase, uint32_t epoch) {
  __shared__ int s_ok;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if ((int)threadIdx.x < a.world) {
    const int peer = threadIdx.x;
    const size_t out_slot = ((size_t)phase * SX_MAX_WORLD + a.rank) * SX_MAX_CTAS + blockIdx.x;
    const size_t in_slot = ((size_t)phase * SX_MAX_WORLD + peer) * SX_MAX_CTAS + blockIdx.x;
    __threadfence_system();
    sx_st_release(a.flags[peer] + out_slot, epoch);
    const long long t0 = clock64();
    while ((int32_t)(sx_ld_acquire(a.flags[a.rank] + in_slot) - epoch) < 0) {
      if (clock64() - t0 > a.wait_cycles) { s_ok = 0; if (a.status) atomicCAS(a.status, 0u, (uint32_t)ST_TIMEOUT_PEER_FLAG); break; }
      __nanosleep(64);
    }
  }
  __syncthreads();
  return s_ok != 0;
}

__global__ void __launch_bounds__(256, 1) state_exchange_kernel(const __grid_constant__ StateExchangeArgs a) {
  const uint32_t epoch = a.words ? *reinterpret_cast<volatile const uint32_t*>(a.words) + 1u : a.epoch;
  const long long n4 = a.numel / 4;
  const long long stride = (long long)gridDim.x * blockDim.x;
  const long long i0 = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  // 1. publish. Each CTA publishes and later reads the SAME index range, so the per-CTA handshake orders them.
  for (long long i = i0; i < n4; i += stride)
    reinterpret_cast<float4*>(a.slot[a.rank])[i] = reinterpret_cast<const float4*>(a.inp)[i];
  const bool ok = sx_handshake(a, 0, epoch);
  // 3. sum the peers this rank needs
  for (long long i = i0; i < n4 && ok; i += stride) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int r = 0; r < a.world; ++r) {
      const bool take = a.mode == 2 || (a.mode == 0 && r < a.rank) || (a.mode == 1 && r > a.rank);
      if (!take) continue;
      const float4 v = __ldcv(reinterpret_cast<const float4*>(a.slot[r]) + i);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    reinterpret_cast<float4*>(a.out)[i] = acc;
  }
  if (ok) sx_handshake(a, 1, epoch);
  if (a.words && threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(a.words + 1, 1u) == gridDim.x - 1) { a.words[1] = 0u; __threadfence(); a.words[0] = epoch; }
  }
}

}  // namespace b200

extern "C" int b200_state_exchange(const b200::StateExchangeArgs* args, int grid, cudaStream_t st) {
  using namespace b200;
  if (args->world < 1 || args->world > SX_MAX_WORLD || grid < 1 || grid > SX_MAX_CTAS || args->numel % 4 != 0) return -1;
  state_exchange_kernel<<<grid, 256, 0, st>>>(*args);
  return (int)cudaGetLastError();
}
extern "C" int b200_state_exchange_flag_words() { return 2 * b200::SX_MAX_WORLD * b200::SX_MAX_CTAS; }
