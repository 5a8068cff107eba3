// M1/M2 building blocks of the mixture-of-experts layers.
//
// The reference's MoE modules compute gate logits and then ignore them, summing ALL experts densely
// (rust-nn src/nn.rs:411-426, 473-487); its top-k router exists as a free function
// (`sparse_topk_route`, src/fused.rs:145-184: top-k, then softmax over the selected logits). Here the
// router really routes:
//   router_fwd : one warp per token - softmax over E experts, top-k by repeated warp arg-max,
//                weights = selected probabilities (optionally renormalised over the k), per-expert
//                token histogram (for the load-balance loss)
//   router_bwd : gradient of the weights (and of the load-balance loss) w.r.t. the logits
//   dispatch   : every (token, choice) claims a slot in its expert's capacity buffer with an atomic
//                counter and copies the token row there. The expert buffers are addressed through a
//                table of base pointers, one per owning rank: with expert parallelism the slot counter
//                and the destination row live in ANOTHER GPU's memory and the claim / copy are a
//                remote atomic and remote stores over NVLink (the all-to-all is these stores).
//   combine    : out[t] = sum_j w[t,j] * y[dest[t,j]]  - rows are pulled from the owning rank's
//                output buffer with peer loads (the reverse all-to-all).
//   combine_bwd / gather_sum : the adjoint permutations.
// No TMA and no cluster multicast is involved; peers are reached with plain ld/st/atomics.
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cstdint>

namespace b200 {

constexpr int MOE_MAX_RANKS = 8;
constexpr int MOE_MAX_PER_LANE = 8;    // experts per lane -> E <= 256
constexpr int MOE_MAX_K = 8;

template <typename T> __device__ __forceinline__ float m_ld(const T* p);
template <> __device__ __forceinline__ float m_ld<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float m_ld<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void m_st(T* p, float v);
template <> __device__ __forceinline__ void m_st<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void m_st<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16(v); }

__device__ __forceinline__ float w_max(float v) { for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o)); return v; }
__device__ __forceinline__ float w_sum(float v) { for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o); return v; }

template <typename T>
__global__ void router_fwd_kernel(const T* __restrict__ logits, int* __restrict__ idx, float* __restrict__ w,
                                  float* __restrict__ probs, int* __restrict__ counts, long long tokens, int E, int k,
                                  int renorm) {
  const long long t = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (t >= tokens) return;
  float p[MOE_MAX_PER_LANE];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < MOE_MAX_PER_LANE; ++i) {
    const int e = lane + 32 * i;
    p[i] = e < E ? m_ld(logits + t * E + e) : -INFINITY;
    mx = fmaxf(mx, p[i]);
  }
  mx = w_max(mx);
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < MOE_MAX_PER_LANE; ++i) { p[i] = (lane + 32 * i) < E ? __expf(p[i] - mx) : 0.f; s += p[i]; }
  s = w_sum(s);
  const float inv = 1.f / s;
#pragma unroll
  for (int i = 0; i < MOE_MAX_PER_LANE; ++i) {
    p[i] *= inv;
    const int e = lane + 32 * i;
    if (e < E) probs[t * E + e] = p[i];
  }
  // top-k: k rounds of (value, index) arg-max; ties resolve to the lower expert index
  float sel_w[MOE_MAX_K]; int sel_i[MOE_MAX_K];
  float wsum = 0.f;
  for (int j = 0; j < k; ++j) {
    float bv = -1.f; int bi = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < MOE_MAX_PER_LANE; ++i) {
      const int e = lane + 32 * i;
      if (e < E && (p[i] > bv || (p[i] == bv && e < bi))) { bv = p[i]; bi = e; }
    }
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    sel_w[j] = bv; sel_i[j] = bi; wsum += bv;
#pragma unroll
    for (int i = 0; i < MOE_MAX_PER_LANE; ++i) if (lane + 32 * i == bi) p[i] = -2.f;   // remove from further rounds
  }
  if (lane == 0) {
    const float rn = renorm ? 1.f / fmaxf(wsum, 1e-20f) : 1.f;
    for (int j = 0; j < k; ++j) {
      idx[t * k + j] = sel_i[j];
      w[t * k + j] = sel_w[j] * rn;
      if (counts) atomicAdd(counts + sel_i[j], 1);
    }
  }
}

// dlogits[t,e] = p_e * (dLdp_e - sum_e' p_e' dLdp_e'),  dLdp_e = aux_g[e] + (e selected ? d(weights)/dp : 0)
template <typename T>
__global__ void router_bwd_kernel(const float* __restrict__ dw, const int* __restrict__ idx, const float* __restrict__ probs,
                                  const float* __restrict__ aux_g, T* __restrict__ dlogits, long long tokens, int E, int k,
                                  int renorm) {
  const long long t = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (t >= tokens) return;
  float p[MOE_MAX_PER_LANE], g[MOE_MAX_PER_LANE];
#pragma unroll
  for (int i = 0; i < MOE_MAX_PER_LANE; ++i) {
    const int e = lane + 32 * i;
    p[i] = e < E ? probs[t * E + e] : 0.f;
    g[i] = (e < E && aux_g) ? aux_g[e] : 0.f;
  }
  float s = 0.f, dot = 0.f;   // s = sum of selected probs, dot = sum_j dw_j * w_j (renormalised weights)
  for (int j = 0; j < k; ++j) { const int e = idx[t * k + j]; s += probs[t * E + e]; }
  if (renorm) { for (int j = 0; j < k; ++j) { const int e = idx[t * k + j]; dot += dw[t * k + j] * probs[t * E + e] / s; } }
  for (int j = 0; j < k; ++j) {
    const int e = idx[t * k + j];
    const float d = renorm ? (dw[t * k + j] - dot) / s : dw[t * k + j];
#pragma unroll
    for (int i = 0; i < MOE_MAX_PER_LANE; ++i) if (lane + 32 * i == e) g[i] += d;
  }
  float pg = 0.f;
#pragma unroll
  for (int i = 0; i < MOE_MAX_PER_LANE; ++i) pg += p[i] * g[i];
  pg = w_sum(pg);
#pragma unroll
  for (int i = 0; i < MOE_MAX_PER_LANE; ++i) {
    const int e = lane + 32 * i;
    if (e < E) m_st(dlogits + t * E + e, p[i] * (g[i] - pg));
  }
}

struct MoeTables {
  void* xbuf[MOE_MAX_RANKS];     // expert input buffers of every rank: [E_local, cap, d]
  int* fill[MOE_MAX_RANKS];      // slot counters of every rank: [E_local]
};

// One warp per (token, choice). dest[t,j] = global row id (owner * E_local * cap + e_local * cap + slot) or -1 if dropped.
__global__ void dispatch_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ idx, int* __restrict__ dest,
                                MoeTables tab, long long tokens, int k, int d, int E_local, int cap) {
  const long long wid = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (wid >= tokens * k) return;
  const long long t = wid / k;
  const int e = idx[wid];
  const int owner = e / E_local, el = e % E_local;
  int slot = 0;
  if (lane == 0) slot = atomicAdd_system(tab.fill[owner] + el, 1);
  slot = __shfl_sync(0xffffffffu, slot, 0);
  if (slot >= cap) { if (lane == 0) dest[wid] = -1; return; }
  if (lane == 0) dest[wid] = (owner * E_local + el) * cap + slot;
  const uint4* src = reinterpret_cast<const uint4*>(x + t * d);
  uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(tab.xbuf[owner]) + ((long long)el * cap + slot) * d);
  for (int i = lane; i < d / 8; i += 32) dst[i] = src[i];
}

struct MoeRead { const void* ybuf[MOE_MAX_RANKS]; };

// out[t,:] = sum_j w[t,j] * ybuf[dest[t,j],:]   (one warp per token; rows may live on a peer)
__global__ void combine_fwd_kernel(MoeRead tab, const int* __restrict__ dest, const float* __restrict__ w,
                                   __nv_bfloat16* __restrict__ out, long long tokens, int k, int d, long long rows_per_rank) {
  const long long t = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (t >= tokens) return;
  for (int c = lane; c < d / 8; c += 32) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int j = 0; j < k; ++j) {
      const int r = dest[t * k + j];
      if (r < 0) continue;
      const float wj = w[t * k + j];
      const int owner = (int)(r / rows_per_rank);
      const long long lr = r % rows_per_rank;
      const uint4 v = *(reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(tab.ybuf[owner]) + lr * d) + c);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
      for (int q = 0; q < 4; ++q) { const float2 f = __bfloat1622float2(h[q]); acc[2 * q] += wj * f.x; acc[2 * q + 1] += wj * f.y; }
    }
    uint4 o;
    __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int q = 0; q < 4; ++q) oh[q] = __floats2bfloat162_rn(acc[2 * q], acc[2 * q + 1]);
    *(reinterpret_cast<uint4*>(out + t * d) + c) = o;
  }
}

struct MoeWrite { void* dybuf[MOE_MAX_RANKS]; };

// dybuf[dest[t,j],:] = w[t,j] * dout[t,:]  (written to the owning rank);  dw[t,j] = <dout[t,:], ybuf[dest[t,j],:]>
__global__ void combine_bwd_kernel(MoeRead ytab, MoeWrite dytab, const int* __restrict__ dest, const float* __restrict__ w,
                                   const __nv_bfloat16* __restrict__ dout, float* __restrict__ dw, long long tokens, int k,
                                   int d, long long rows_per_rank) {
  const long long wid = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (wid >= tokens * k) return;
  const long long t = wid / k;
  const int r = dest[wid];
  if (r < 0) { if (lane == 0) dw[wid] = 0.f; return; }
  const float wj = w[wid];
  const int owner = (int)(r / rows_per_rank);
  const long long lr = r % rows_per_rank;
  const uint4* gsrc = reinterpret_cast<const uint4*>(dout + t * d);
  const uint4* ysrc = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(ytab.ybuf[owner]) + lr * d);
  uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(dytab.dybuf[owner]) + lr * d);
  float dot = 0.f;
  for (int c = lane; c < d / 8; c += 32) {
    const uint4 g = gsrc[c], y = ysrc[c];
    const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&g);
    const __nv_bfloat162* yh = reinterpret_cast<const __nv_bfloat162*>(&y);
    uint4 o; __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float2 gf = __bfloat1622float2(gh[q]), yf = __bfloat1622float2(yh[q]);
      dot += gf.x * yf.x + gf.y * yf.y;
      oh[q] = __floats2bfloat162_rn(gf.x * wj, gf.y * wj);
    }
    dst[c] = o;
  }
  dot = w_sum(dot);
  if (lane == 0) dw[wid] = dot;
}

// dx[t,:] = sum_j dxbuf[dest[t,j],:]   (adjoint of dispatch; rows pulled from the owning rank)
__global__ void gather_sum_kernel(MoeRead tab, const int* __restrict__ dest, __nv_bfloat16* __restrict__ dx,
                                  long long tokens, int k, int d, long long rows_per_rank) {
  const long long t = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (t >= tokens) return;
  for (int c = lane; c < d / 8; c += 32) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int j = 0; j < k; ++j) {
      const int r = dest[t * k + j];
      if (r < 0) continue;
      const int owner = (int)(r / rows_per_rank);
      const long long lr = r % rows_per_rank;
      const uint4 v = *(reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(tab.ybuf[owner]) + lr * d) + c);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
      for (int q = 0; q < 4; ++q) { const float2 f = __bfloat1622float2(h[q]); acc[2 * q] += f.x; acc[2 * q + 1] += f.y; }
    }
    uint4 o; __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int q = 0; q < 4; ++q) oh[q] = __floats2bfloat162_rn(acc[2 * q], acc[2 * q + 1]);
    *(reinterpret_cast<uint4*>(dx + t * d) + c) = o;
  }
}

// Cross-rank barrier on the stream: everything this rank launched before it is complete and visible to the peers
// once they leave it, and nothing launched after it starts before every rank has arrived. Replaces a host barrier
// between the dispatch / expert-GEMM / combine phases, so an expert-parallel step can be captured into a CUDA graph.
// The epoch is a device word bumped here (one thread block, one launch at a time per context).
struct EpBarrierArgs {
  uint32_t* flags[MOE_MAX_RANKS];   // every rank's flag words [MOE_MAX_RANKS] (peer-mapped): slot r is written by rank r
  uint32_t* words;                  // local: [0] barriers passed so far
  int rank, world;
  long long wait_cycles;
  uint32_t* status;
};

__global__ void ep_barrier_kernel(const EpBarrierArgs a) {
  const uint32_t epoch = a.words[0] + 1u;
  if ((int)threadIdx.x < a.world) {
    const int peer = threadIdx.x;
    __threadfence_system();
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(a.flags[peer] + a.rank), "r"(epoch) : "memory");
    const long long t0 = clock64();
    for (;;) {
      uint32_t v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(a.flags[a.rank] + peer) : "memory");
      if ((int32_t)(v - epoch) >= 0) break;
      if (clock64() - t0 > a.wait_cycles) { if (a.status) atomicCAS(a.status, 0u, 5u); break; }
      __nanosleep(64);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) { __threadfence_system(); a.words[0] = epoch; }
}

static inline unsigned warps_grid(long long warps) { return (unsigned)((warps * 32 + 255) / 256); }

}  // namespace b200

using namespace b200;

extern "C" {

int b200_router_fwd(const void* logits, int* idx, float* w, float* probs, int* counts, long long tokens, int E, int k,
                    int renorm, int is_bf16, cudaStream_t st) {
  if (tokens <= 0) return 0;
  if (E > 32 * MOE_MAX_PER_LANE || k > MOE_MAX_K || k > E || k < 1) return -1;
  if (is_bf16) router_fwd_kernel<__nv_bfloat16><<<warps_grid(tokens), 256, 0, st>>>((const __nv_bfloat16*)logits, idx, w, probs, counts, tokens, E, k, renorm);
  else router_fwd_kernel<float><<<warps_grid(tokens), 256, 0, st>>>((const float*)logits, idx, w, probs, counts, tokens, E, k, renorm);
  return (int)cudaGetLastError();
}

int b200_router_bwd(const float* dw, const int* idx, const float* probs, const float* aux_g, void* dlogits, long long tokens,
                    int E, int k, int renorm, int is_bf16, cudaStream_t st) {
  if (tokens <= 0) return 0;
  if (E > 32 * MOE_MAX_PER_LANE || k > MOE_MAX_K) return -1;
  if (is_bf16) router_bwd_kernel<__nv_bfloat16><<<warps_grid(tokens), 256, 0, st>>>(dw, idx, probs, aux_g, (__nv_bfloat16*)dlogits, tokens, E, k, renorm);
  else router_bwd_kernel<float><<<warps_grid(tokens), 256, 0, st>>>(dw, idx, probs, aux_g, (float*)dlogits, tokens, E, k, renorm);
  return (int)cudaGetLastError();
}

// xbuf / fill: arrays of `world` base pointers (this rank's view of every rank's buffers)
int b200_moe_dispatch(const void* x, const int* idx, int* dest, void* const* xbuf, int* const* fill, int world,
                      long long tokens, int k, int d, int E_local, int cap, cudaStream_t st) {
  if (tokens <= 0) return 0;
  if (world < 1 || world > MOE_MAX_RANKS || d % 8) return -1;
  MoeTables tab;
  for (int r = 0; r < world; ++r) { tab.xbuf[r] = xbuf[r]; tab.fill[r] = fill[r]; }
  dispatch_kernel<<<warps_grid(tokens * k), 256, 0, st>>>((const __nv_bfloat16*)x, idx, dest, tab, tokens, k, d, E_local, cap);
  return (int)cudaGetLastError();
}

int b200_moe_combine_fwd(void* const* ybuf, int world, const int* dest, const float* w, void* out, long long tokens, int k,
                         int d, long long rows_per_rank, cudaStream_t st) {
  if (tokens <= 0) return 0;
  if (world < 1 || world > MOE_MAX_RANKS || d % 8) return -1;
  MoeRead tab; for (int r = 0; r < world; ++r) tab.ybuf[r] = ybuf[r];
  combine_fwd_kernel<<<warps_grid(tokens), 256, 0, st>>>(tab, dest, w, (__nv_bfloat16*)out, tokens, k, d, rows_per_rank);
  return (int)cudaGetLastError();
}

int b200_moe_combine_bwd(void* const* ybuf, void* const* dybuf, int world, const int* dest, const float* w, const void* dout,
                         float* dw, long long tokens, int k, int d, long long rows_per_rank, cudaStream_t st) {
  if (tokens <= 0) return 0;
  if (world < 1 || world > MOE_MAX_RANKS || d % 8) return -1;
  MoeRead yt; MoeWrite dt;
  for (int r = 0; r < world; ++r) { yt.ybuf[r] = ybuf[r]; dt.dybuf[r] = dybuf[r]; }
  combine_bwd_kernel<<<warps_grid(tokens * k), 256, 0, st>>>(yt, dt, dest, w, (const __nv_bfloat16*)dout, dw, tokens, k, d, rows_per_rank);
  return (int)cudaGetLastError();
}

int b200_ep_barrier(uint32_t* const* flags, int world, int rank, uint32_t* words, long long wait_cycles, uint32_t* status, cudaStream_t st) {
  if (world < 1 || world > MOE_MAX_RANKS || rank < 0 || rank >= world) return -1;
  EpBarrierArgs a;
  for (int r = 0; r < world; ++r) a.flags[r] = flags[r];
  a.words = words; a.rank = rank; a.world = world; a.wait_cycles = wait_cycles; a.status = status;
  ep_barrier_kernel<<<1, 32, 0, st>>>(a);
  return (int)cudaGetLastError();
}

int b200_moe_gather_sum(void* const* buf, int world, const int* dest, void* dx, long long tokens, int k, int d,
                        long long rows_per_rank, cudaStream_t st) {
  if (tokens <= 0) return 0;
  if (world < 1 || world > MOE_MAX_RANKS || d % 8) return -1;
  MoeRead tab; for (int r = 0; r < world; ++r) tab.ybuf[r] = buf[r];
  gather_sum_kernel<<<warps_grid(tokens), 256, 0, st>>>(tab, dest, (__nv_bfloat16*)dx, tokens, k, d, rows_per_rank);
  return (int)cudaGetLastError();
}

}  // extern "C"
