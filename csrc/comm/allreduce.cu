// Small all-reduce over NVLink peer memory (sum; fp32 or bf16 in, bf16 out), for the replicated
// activations of a tensor-parallel block: the [tokens, dt_rank + 2*d_state] output of Mamba's
// row-parallel x-projection and its gradient. The reference has no tensor parallelism (its only
// multi-worker path is the simulated gradient all-reduce, rust-nn src/distributed.rs:54-124).
//
// Two-shot, one kernel:
//   1. publish: copy the local partial into this rank's peer-mapped input buffer
//   2. handshake 0, then reduce the slice this rank owns (1/world of the array) from every peer's
//      input buffer in rank order, fp32 accumulation, and keep the bf16 result in this rank's
//      peer-mapped result buffer - each element crosses NVLink (world-1)/world times here
//   3. handshake 1, then gather every rank's slice from its result buffer into the local output
//   4. handshake 2: nobody overwrites a buffer that a peer still reads
// Every loop walks a slice with the same (CTA, thread) -> element mapping, so CTA j only ever reads
// what CTA j of a peer wrote and a per-CTA flag exchange is enough. Each element is reduced by exactly
// one rank, so all ranks end with identical bits. Waits are bounded (clock budget -> status word).
// The call epoch is a device word advanced by the last CTA to retire (CUDA-graph replay safe).
#include <cuda_runtime.h>
#include <cstdint>
#include "../common/ptx.cuh"

namespace b200 {

constexpr int AR_MAX_WORLD = 8;
constexpr int AR_MAX_CTAS = 64;
constexpr int AR_THREADS = 512;

struct AllReduceArgs {
  void* in_sym[AR_MAX_WORLD];       // every rank's input buffer (peer-mapped), numel elements of the input type
  void* red_sym[AR_MAX_WORLD];      // every rank's result buffer (peer-mapped), numel bf16 (only the owner's slice is used)
  uint32_t* flags[AR_MAX_WORLD];    // [3][AR_MAX_WORLD][AR_MAX_CTAS] words per rank (peer-mapped)
  const void* inp;                  // local partial [numel]
  void* out;                        // local result [numel] bf16
  long long numel;                  // multiple of 8 * world
  int rank, world, in_bf16;
  long long wait_cycles;
  uint32_t* status;
  uint32_t* words;                  // local: [0] calls so far, [1] retired CTAs
};

__device__ __forceinline__ bool ar_handshake(const AllReduceArgs& a, int phase, uint32_t epoch) {
  __shared__ int s_ok;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if ((int)threadIdx.x < a.world) {
    const int peer = threadIdx.x;
    const size_t out_slot = ((size_t)phase * AR_MAX_WORLD + a.rank) * AR_MAX_CTAS + blockIdx.x;
    const size_t in_slot = ((size_t)phase * AR_MAX_WORLD + peer) * AR_MAX_CTAS + blockIdx.x;
    __threadfence_system();
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(a.flags[peer] + out_slot), "r"(epoch) : "memory");
    const long long t0 = clock64();
    for (;;) {
      uint32_t v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(a.flags[a.rank] + in_slot) : "memory");
      if ((int32_t)(v - epoch) >= 0) break;
      if (clock64() - t0 > a.wait_cycles) { s_ok = 0; if (a.status) atomicCAS(a.status, 0u, (uint32_t)ST_TIMEOUT_PEER_FLAG); break; }
      __nanosleep(64);
    }
  }
  __syncthreads();
  return s_ok != 0;
}

// 8 elements per thread-iteration: 32 bytes of fp32 or 16 bytes of bf16 in, 16 bytes of bf16 out
__device__ __forceinline__ void load8(const void* base, long long i8, int bf16, float* v) {
  if (bf16) {
    const uint4 u = __ldcv(reinterpret_cast<const uint4*>(base) + i8);
    const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y; v[4] = c.x; v[5] = c.y; v[6] = d.x; v[7] = d.y;
  } else {
    const float4 x = __ldcv(reinterpret_cast<const float4*>(base) + 2 * i8), y = __ldcv(reinterpret_cast<const float4*>(base) + 2 * i8 + 1);
    v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w; v[4] = y.x; v[5] = y.y; v[6] = y.z; v[7] = y.w;
  }
}

__global__ void __launch_bounds__(AR_THREADS, 1) allreduce_kernel(const __grid_constant__ AllReduceArgs a) {
  const uint32_t epoch = *reinterpret_cast<volatile const uint32_t*>(a.words) + 1u;
  const long long n8 = a.numel / 8, slice = n8 / a.world;
  const long long x0 = (long long)blockIdx.x * blockDim.x + threadIdx.x, stride = (long long)gridDim.x * blockDim.x;
  // 1. publish (slice by slice, with the mapping the readers use)
  for (int s = 0; s < a.world; ++s)
    for (long long x = x0; x < slice; x += stride) {
      const long long i8 = (long long)s * slice + x;
      if (a.in_bf16) {
        reinterpret_cast<uint4*>(a.in_sym[a.rank])[i8] = reinterpret_cast<const uint4*>(a.inp)[i8];
      } else {
        reinterpret_cast<float4*>(a.in_sym[a.rank])[2 * i8] = reinterpret_cast<const float4*>(a.inp)[2 * i8];
        reinterpret_cast<float4*>(a.in_sym[a.rank])[2 * i8 + 1] = reinterpret_cast<const float4*>(a.inp)[2 * i8 + 1];
      }
    }
  bool ok = ar_handshake(a, 0, epoch);
  // 2. reduce the owned slice
  for (long long x = x0; x < slice && ok; x += stride) {
    const long long i8 = (long long)a.rank * slice + x;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int p = 0; p < a.world; ++p) {
      float v[8];
      load8(a.in_sym[p], i8, a.in_bf16, v);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += v[j];
    }
    reinterpret_cast<uint4*>(a.red_sym[a.rank])[i8] =
        make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]), pack_bf16x2(acc[4], acc[5]), pack_bf16x2(acc[6], acc[7]));
  }
  ok = ok && ar_handshake(a, 1, epoch);
  // 3. gather all slices
  for (int s = 0; s < a.world && ok; ++s) {
    const int p = (a.rank + s) % a.world;
    for (long long x = x0; x < slice; x += stride) {
      const long long i8 = (long long)p * slice + x;
      reinterpret_cast<uint4*>(a.out)[i8] = __ldcv(reinterpret_cast<const uint4*>(a.red_sym[p]) + i8);
    }
  }
  if (ok) ar_handshake(a, 2, epoch);
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(a.words + 1, 1u) == gridDim.x - 1) { a.words[1] = 0u; __threadfence(); a.words[0] = epoch; }
  }
}

}  // namespace b200

extern "C" int b200_allreduce_bf16(const b200::AllReduceArgs* args, int grid, cudaStream_t st) {
  using namespace b200;
  if (args->world < 1 || args->world > AR_MAX_WORLD || grid < 1 || grid > AR_MAX_CTAS) return -1;
  if (args->numel % (8LL * args->world) != 0) return -2;
  allreduce_kernel<<<grid, AR_THREADS, 0, st>>>(*args);
  return (int)cudaGetLastError();
}
extern "C" int b200_allreduce_flag_words() { return 3 * b200::AR_MAX_WORLD * b200::AR_MAX_CTAS; }
