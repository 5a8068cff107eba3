// O1c: data-parallel gradient reduce-scatter fused with the scale/cast, the Adam update and the
// all-gather of the updated bf16 weights - ONE kernel per step, over NVLink peer memory.
//
// The reference's data-parallel step flattens all gradients into one bucket, sums the buckets of all
// workers, divides by the world size, writes the result back and then runs the optimizer
// (rust-nn src/distributed.rs:140-196, 472-503 - an in-process simulation). Here every rank owns the
// shard [rank*n/W, (rank+1)*n/W) of the flat parameter space:
//   1. flag handshake (st.release.sys / ld.acquire.sys, per-CTA slots in every peer's symmetric
//      flag area) - "all ranks have finished backward";
//   2. for its shard: g = (1/W) * sum_p grad_p[i], read straight from the peers' gradient buffers
//      (P2P loads, or one multimem.ld_reduce through the NVSwitch when a multicast mapping is given);
//      Adam on the fp32 master shard; the new weights are cast to bf16 and stored into EVERY rank's
//      shadow-weight buffer (P2P stores, or one multimem.st);
//   3. second handshake - "all shards have landed everywhere", so the next forward may start.
// No TMA is involved (and no cluster multicast anywhere). Waits are bounded by a clock budget; on
// expiry the kernel records ST_TIMEOUT_PEER_FLAG and returns.
#include "../common/ptx.cuh"

namespace b200 {

constexpr int DP_MAX_WORLD = 8;
constexpr int DP_MAX_CTAS = 160;

struct DpFusedArgs {
  float* grad[DP_MAX_WORLD];              // flat fp32 gradient buffer of every rank (peer-mapped)
  __nv_bfloat16* shadow[DP_MAX_WORLD];    // flat bf16 weight buffer of every rank (peer-mapped)
  uint32_t* flags[DP_MAX_WORLD];          // [2][DP_MAX_WORLD][DP_MAX_CTAS] words per rank (peer-mapped)
  float* grad_mc;                         // multicast address of the gradient buffers (or null)
  __nv_bfloat16* shadow_mc;               // multicast address of the shadow buffers (or null)
  float* master; float* m; float* v;      // local flat fp32 buffers (full length, only the shard is touched)
  long long n;                            // flat length, multiple of 8*world
  int rank, world;
  float lr, b1, b2, eps, weight_decay; int torch_form;
  const float* step_ptr;                  // device step counter (also the handshake epoch)
  const float* grad_scale_ptr;            // optional clip coefficient
  uint32_t* status;
  long long wait_cycles;                  // clock64 budget for one handshake
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float4 ld_peer_f4(const float* p) {
  float4 v;
  asm volatile("ld.volatile.global.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float4 multimem_ld_reduce_f4(const float* p) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void multimem_st_b128(void* p, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};"
               ::"l"(p), "f"(__uint_as_float(v.x)), "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)), "f"(__uint_as_float(v.w)) : "memory");
}

// Per-CTA all-to-all handshake. Thread t < world signals peer t and waits for peer t.
__device__ __forceinline__ bool handshake(const DpFusedArgs& a, int phase, uint32_t epoch) {
  __shared__ int s_ok;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if ((int)threadIdx.x < a.world) {
    const int peer = threadIdx.x;
    const size_t slot_out = ((size_t)phase * DP_MAX_WORLD + a.rank) * DP_MAX_CTAS + blockIdx.x;   // my slot at the peer
    const size_t slot_in = ((size_t)phase * DP_MAX_WORLD + peer) * DP_MAX_CTAS + blockIdx.x;      // peer's slot here
    __threadfence_system();
    st_release_sys(a.flags[peer] + slot_out, epoch);
    const long long t0 = clock64();
    bool ok = true;
    while (ld_acquire_sys(a.flags[a.rank] + slot_in) < epoch) {
      if (clock64() - t0 > a.wait_cycles) { ok = false; break; }
      __nanosleep(64);
    }
    if (!ok) { s_ok = 0; if (a.status) atomicCAS(a.status, 0u, (uint32_t)ST_TIMEOUT_PEER_FLAG); }
  }
  __syncthreads();
  return s_ok != 0;
}

__global__ void __launch_bounds__(512, 1) dp_fused_adam_kernel(const __grid_constant__ DpFusedArgs a) {
  const uint32_t epoch = (uint32_t)(*a.step_ptr) + 1u;
  if (!handshake(a, 0, epoch)) return;

  const float t = *a.step_ptr + 1.f;
  const float bc1 = 1.f - powf(a.b1, t), bc2 = 1.f - powf(a.b2, t);
  const float lr_t = a.torch_form ? a.lr / bc1 : a.lr * sqrtf(bc2) / bc1;
  const float c2 = a.torch_form ? rsqrtf(bc2) : 1.f;
  const float gs = (a.grad_scale_ptr ? *a.grad_scale_ptr : 1.f) / (float)a.world;
  const float ob1 = 1.f - a.b1, ob2 = 1.f - a.b2;

  const long long shard = a.n / a.world;
  const long long base = shard * a.rank;
  const long long n8 = shard / 8;                       // 8 elements per thread-iteration (16 B of bf16 out)
  for (long long i8 = blockIdx.x * (long long)blockDim.x + threadIdx.x; i8 < n8; i8 += (long long)gridDim.x * blockDim.x) {
    const long long i = base + i8 * 8;
    float g[8];
    if (a.grad_mc) {
      float4 x = multimem_ld_reduce_f4(a.grad_mc + i), y = multimem_ld_reduce_f4(a.grad_mc + i + 4);
      g[0] = x.x; g[1] = x.y; g[2] = x.z; g[3] = x.w; g[4] = y.x; g[5] = y.y; g[6] = y.z; g[7] = y.w;
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) g[j] = 0.f;
      for (int p = 0; p < a.world; ++p) {
        const int peer = (a.rank + p) % a.world;        // start at self, stagger the peers
        float4 x = ld_peer_f4(a.grad[peer] + i), y = ld_peer_f4(a.grad[peer] + i + 4);
        g[0] += x.x; g[1] += x.y; g[2] += x.z; g[3] += x.w; g[4] += y.x; g[5] += y.y; g[6] += y.z; g[7] += y.w;
      }
    }
    float pm[8], mm[8], vv[8];
    *reinterpret_cast<float4*>(pm) = *reinterpret_cast<const float4*>(a.master + i);
    *reinterpret_cast<float4*>(pm + 4) = *reinterpret_cast<const float4*>(a.master + i + 4);
    *reinterpret_cast<float4*>(mm) = *reinterpret_cast<const float4*>(a.m + i);
    *reinterpret_cast<float4*>(mm + 4) = *reinterpret_cast<const float4*>(a.m + i + 4);
    *reinterpret_cast<float4*>(vv) = *reinterpret_cast<const float4*>(a.v + i);
    *reinterpret_cast<float4*>(vv + 4) = *reinterpret_cast<const float4*>(a.v + i + 4);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float gr = g[j] * gs;
      if (a.weight_decay != 0.f) pm[j] -= a.lr * a.weight_decay * pm[j];
      mm[j] = a.b1 * mm[j] + ob1 * gr;
      vv[j] = a.b2 * vv[j] + ob2 * gr * gr;
      pm[j] -= lr_t * mm[j] / (sqrtf(vv[j]) * c2 + a.eps);
    }
    *reinterpret_cast<float4*>(a.master + i) = *reinterpret_cast<float4*>(pm);
    *reinterpret_cast<float4*>(a.master + i + 4) = *reinterpret_cast<float4*>(pm + 4);
    *reinterpret_cast<float4*>(a.m + i) = *reinterpret_cast<float4*>(mm);
    *reinterpret_cast<float4*>(a.m + i + 4) = *reinterpret_cast<float4*>(mm + 4);
    *reinterpret_cast<float4*>(a.v + i) = *reinterpret_cast<float4*>(vv);
    *reinterpret_cast<float4*>(a.v + i + 4) = *reinterpret_cast<float4*>(vv + 4);
    const uint4 packed = make_uint4(pack_bf16x2(pm[0], pm[1]), pack_bf16x2(pm[2], pm[3]), pack_bf16x2(pm[4], pm[5]), pack_bf16x2(pm[6], pm[7]));
    if (a.shadow_mc) {
      multimem_st_b128(a.shadow_mc + i, packed);
    } else {
      for (int p = 0; p < a.world; ++p) {
        const int peer = (a.rank + p) % a.world;
        *reinterpret_cast<uint4*>(a.shadow[peer] + i) = packed;
      }
    }
  }
  __threadfence_system();
  handshake(a, 1, epoch);
}

}  // namespace b200

// The argument block is passed by value (it holds the peer pointers). `grid` must be identical on
// all ranks and at most DP_MAX_CTAS (<= number of SMs so that every CTA is resident).
extern "C" int b200_dp_fused_adam(const b200::DpFusedArgs* args, int grid, cudaStream_t st) {
  using namespace b200;
  if (args->world < 1 || args->world > DP_MAX_WORLD || grid < 1 || grid > DP_MAX_CTAS) return -1;
  if (args->n % (8LL * args->world) != 0) return -2;
  dp_fused_adam_kernel<<<grid, 512, 0, st>>>(*args);
  return (int)cudaGetLastError();
}

extern "C" int b200_dp_flag_words() { return 2 * b200::DP_MAX_WORLD * b200::DP_MAX_CTAS; }
