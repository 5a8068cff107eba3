// O1c / O2c: data-parallel gradient reduce-scatter fused with the scale/cast, the optimizer update and
// the all-gather of the updated bf16 weights, over NVLink peer memory.
//
// The reference's data-parallel step flattens all gradients into one bucket, sums the buckets of all
// workers, divides by the world size, clips by the global norm of the AVERAGED gradient, writes the
// result back and then runs the optimizer (rust-nn src/distributed.rs:140-196, 472-523 - an in-process
// simulation). Here the flat parameter space has two parts:
//
//   * the SHARDED range, cut into buckets [begin, end). Inside a bucket rank r owns the slice
//     [begin + r*len/W, begin + (r+1)*len/W): it sums that slice of every peer's gradient buffer
//     (P2P loads, or one multimem.ld_reduce through the NVSwitch), updates its fp32 master weights and
//     optimizer state there, and stores the new bf16 weights into EVERY rank's shadow buffer (P2P
//     stores, or one multimem.st). A bucket is one launch, so buckets whose gradients are complete can
//     run on a side stream while backward is still producing the others.
//   * the REPLICATED range (biases, norm gains, small tables: everything the forward reads in fp32).
//     Every rank reduces it from all peers in the SAME order and applies the same update, so the fp32
//     master values of these parameters are bit-identical on all ranks and nothing has to be sent back.
//
// Three kernels:
//   dp_fused_adam_kernel   one pass: handshake, reduce + Adam + all-gather, handshake. Used when nothing
//                          needs a norm of the reduced gradient.
//   dp_reduce_kernel       pass 1 of 2: handshake, reduce the owned slice IN PLACE in this rank's own
//                          gradient buffer (peers never read that slice), accumulate the sum of squares
//                          per parameter tensor (Muon) or in total (clipping) into a peer-mapped table.
//   dp_update_kernel       pass 2 of 2: handshake (so every rank's table is complete), combine the tables
//                          of all ranks in a fixed order, then Adam with the global-norm clip coefficient
//                          (src/distributed.rs:507-523: clip AFTER averaging) or the reference's Muon
//                          (gradient / per-tensor RMS, momentum SGD, src/optim.rs:284-307), all-gather,
//                          handshake.
//
// The handshake epoch is a device word of its own that each launch bumps when its last CTA retires. It is
// not optimizer state: restoring a checkpoint (or the snapshot a CUDA-graph capture takes around its
// warm-up steps) rewinds the Adam step counter but never the epoch, so the flags in peer memory can
// never be ahead of it. No TMA is involved (and no cluster multicast anywhere). Waits are bounded by a
// clock budget; on expiry the kernel records ST_TIMEOUT_PEER_FLAG and returns.
#include "../common/ptx.cuh"

namespace b200 {

constexpr int DP_MAX_WORLD = 8;
constexpr int DP_MAX_CTAS = 160;
constexpr int DP_THREADS = 512;

struct DpFusedArgs {
  float* grad[DP_MAX_WORLD];              // flat fp32 gradient buffer of every rank (peer-mapped)
  __nv_bfloat16* shadow[DP_MAX_WORLD];    // flat bf16 weight buffer of every rank (peer-mapped)
  uint32_t* flags[DP_MAX_WORLD];          // [2][DP_MAX_WORLD][DP_MAX_CTAS] words per rank (peer-mapped)
  float* partial[DP_MAX_WORLD];           // [2][max(nseg,1)] sums of squares per rank (peer-mapped), two-pass only
  float* grad_mc;                         // multicast address of the gradient buffers (or null)
  __nv_bfloat16* shadow_mc;               // multicast address of the shadow buffers (or null)
  float* master; float* m; float* v;      // local flat fp32 buffers (full length)
  long long begin, end;                   // sharded bucket of this launch; (end - begin) % (8 * world) == 0
  long long rep_begin, rep_end;           // replicated range handled by this launch (empty if equal)
  int rank, world;
  float lr, b1, b2, eps, weight_decay; int torch_form;
  int rule;                               // 0 Adam, 1 Muon (momentum = b1, buffer = m)
  int scale_mode;                         // two-pass: 1 = clip by global norm, 2 = divide by per-tensor RMS
  const float* step_ptr;                  // optimizer step counter (bias correction)
  const float* grad_scale_ptr;            // optional extra gradient multiplier
  uint32_t* words;                        // local: [0] handshake epoch, [1] retired-CTA counter, [2] two-pass counter
  uint32_t* status;
  long long wait_cycles;                  // clock64 budget for one handshake
  const long long* seg_off;               // [nseg][2] begin/end of every parameter tensor in the flat space, ascending
  const int* blk_seg;                     // index of the tensor that holds (or follows) element 1024*j
  int nseg, first_rep_seg;                // tensors with index >= first_rep_seg live in the replicated range
  float* red_rep;                         // local [rep_end - rep_begin]: reduced gradient of the replicated range
  float* rep_sumsq;                       // local [nseg]: sum of squares of the reduced replicated tensors
  float clip_max_norm;                    // scale_mode 1: > 0 clips, <= 0 only reports the norm
  float* norm_out;                        // optional: the global gradient norm (written by CTA 0)
  int bump_pass;                          // 1: this launch closes a two-pass step (bump words[2])
  float red_scale;                        // multiplies the summed gradient: 1/world (mean over ranks) or 1 (sum)
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
__device__ __forceinline__ float ld_peer_f1(const float* p) {
  float v;
  asm volatile("ld.volatile.global.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
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
    // signed distance: correct across the 2^32 wrap of the epoch
    while ((int32_t)(ld_acquire_sys(a.flags[a.rank] + slot_in) - epoch) < 0) {
      if (clock64() - t0 > a.wait_cycles) { ok = false; break; }
      __nanosleep(64);
    }
    if (!ok) { s_ok = 0; if (a.status) atomicCAS(a.status, 0u, (uint32_t)ST_TIMEOUT_PEER_FLAG); }
  }
  __syncthreads();
  return s_ok != 0;
}

// Every CTA calls this once, after its last use of the epoch: the CTA that retires last advances the epoch.
__device__ __forceinline__ void retire(const DpFusedArgs& a) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const uint32_t old = atomicAdd(a.words + 1, 1u);
    if (old == gridDim.x - 1) {
      a.words[1] = 0u;
      if (a.bump_pass) a.words[2] += 1u;
      __threadfence();
      a.words[0] += 1u;
    }
  }
}

struct Hyper { float lr_t, c2, gs, ob1, ob2; };

__device__ __forceinline__ Hyper make_hyper(const DpFusedArgs& a) {
  Hyper h;
  const float t = *a.step_ptr + 1.f;
  const float bc1 = 1.f - powf(a.b1, t), bc2 = 1.f - powf(a.b2, t);
  h.lr_t = a.torch_form ? a.lr / bc1 : a.lr * sqrtf(bc2) / bc1;
  h.c2 = a.torch_form ? rsqrtf(bc2) : 1.f;
  h.gs = (a.grad_scale_ptr ? *a.grad_scale_ptr : 1.f);
  h.ob1 = 1.f - a.b1; h.ob2 = 1.f - a.b2;
  return h;
}

// One parameter element. `gr` is the averaged (and scaled) gradient.
__device__ __forceinline__ void apply_rule(const DpFusedArgs& a, const Hyper& h, float gr, float& p, float& m, float& v) {
  if (a.rule == 0) {
    if (a.weight_decay != 0.f) p -= a.lr * a.weight_decay * p;
    m = a.b1 * m + h.ob1 * gr;
    v = a.b2 * v + h.ob2 * gr * gr;
    p -= h.lr_t * m / (sqrtf(v) * h.c2 + a.eps);
  } else {
    m = a.b1 * m + gr;            // Muon: gr has been divided by the tensor's RMS already
    p -= a.lr * m;
  }
}

// 8 consecutive elements at flat index i (i % 8 == 0): load state, apply, store state, return the bf16 pack.
__device__ __forceinline__ uint4 update8(const DpFusedArgs& a, const Hyper& h, long long i, const float* gr) {
  float pm[8], mm[8], vv[8];
  *reinterpret_cast<float4*>(pm) = *reinterpret_cast<const float4*>(a.master + i);
  *reinterpret_cast<float4*>(pm + 4) = *reinterpret_cast<const float4*>(a.master + i + 4);
  *reinterpret_cast<float4*>(mm) = *reinterpret_cast<const float4*>(a.m + i);
  *reinterpret_cast<float4*>(mm + 4) = *reinterpret_cast<const float4*>(a.m + i + 4);
  if (a.rule == 0) {
    *reinterpret_cast<float4*>(vv) = *reinterpret_cast<const float4*>(a.v + i);
    *reinterpret_cast<float4*>(vv + 4) = *reinterpret_cast<const float4*>(a.v + i + 4);
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) apply_rule(a, h, gr[j], pm[j], mm[j], vv[j]);
  *reinterpret_cast<float4*>(a.master + i) = *reinterpret_cast<float4*>(pm);
  *reinterpret_cast<float4*>(a.master + i + 4) = *reinterpret_cast<float4*>(pm + 4);
  *reinterpret_cast<float4*>(a.m + i) = *reinterpret_cast<float4*>(mm);
  *reinterpret_cast<float4*>(a.m + i + 4) = *reinterpret_cast<float4*>(mm + 4);
  if (a.rule == 0) {
    *reinterpret_cast<float4*>(a.v + i) = *reinterpret_cast<float4*>(vv);
    *reinterpret_cast<float4*>(a.v + i + 4) = *reinterpret_cast<float4*>(vv + 4);
  }
  return make_uint4(pack_bf16x2(pm[0], pm[1]), pack_bf16x2(pm[2], pm[3]), pack_bf16x2(pm[4], pm[5]), pack_bf16x2(pm[6], pm[7]));
}

__device__ __forceinline__ void publish8(const DpFusedArgs& a, long long i, uint4 packed) {
  if (a.shadow_mc) {
    multimem_st_b128(a.shadow_mc + i, packed);
  } else {
    for (int p = 0; p < a.world; ++p) {
      const int peer = (a.rank + p) % a.world;         // start at self, stagger the peers
      *reinterpret_cast<uint4*>(a.shadow[peer] + i) = packed;
    }
  }
}

// Sum of the peers' gradients for 8 elements of the owned slice (any order: only this rank computes it).
__device__ __forceinline__ void reduce8(const DpFusedArgs& a, long long i, float* g) {
  if (a.grad_mc) {
    float4 x = multimem_ld_reduce_f4(a.grad_mc + i), y = multimem_ld_reduce_f4(a.grad_mc + i + 4);
    g[0] = x.x; g[1] = x.y; g[2] = x.z; g[3] = x.w; g[4] = y.x; g[5] = y.y; g[6] = y.z; g[7] = y.w;
    return;
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) g[j] = 0.f;
  for (int p = 0; p < a.world; ++p) {
    const int peer = (a.rank + p) % a.world;
    float4 x = ld_peer_f4(a.grad[peer] + i), y = ld_peer_f4(a.grad[peer] + i + 4);
    g[0] += x.x; g[1] += x.y; g[2] += x.z; g[3] += x.w; g[4] += y.x; g[5] += y.y; g[6] += y.z; g[7] += y.w;
  }
}

// Sum over the ranks in rank order 0..W-1: every rank gets the same bits (replicated range).
__device__ __forceinline__ float reduce1_ordered(const DpFusedArgs& a, long long i) {
  float g = 0.f;
  for (int p = 0; p < a.world; ++p) g += ld_peer_f1(a.grad[p] + i);
  return g;
}

// ------------------------------------------------------------------------------------------------ one pass
__global__ void __launch_bounds__(DP_THREADS, 1) dp_fused_adam_kernel(const __grid_constant__ DpFusedArgs a) {
  const uint32_t epoch = a.words[0] + 1u;
  if (!handshake(a, 0, epoch)) { retire(a); return; }
  const Hyper h = make_hyper(a);
  const float gs = h.gs * a.red_scale;

  const long long shard = (a.end - a.begin) / a.world;
  const long long base = a.begin + shard * a.rank;
  const long long n8 = shard / 8;                       // 8 elements per thread-iteration (16 B of bf16 out)
  for (long long i8 = blockIdx.x * (long long)blockDim.x + threadIdx.x; i8 < n8; i8 += (long long)gridDim.x * blockDim.x) {
    const long long i = base + i8 * 8;
    float g[8];
    reduce8(a, i, g);
#pragma unroll
    for (int j = 0; j < 8; ++j) g[j] *= gs;
    publish8(a, i, update8(a, h, i, g));
  }
  // replicated range: identical arithmetic on every rank, local shadow only
  for (long long i = a.rep_begin + blockIdx.x * (long long)blockDim.x + threadIdx.x; i < a.rep_end; i += (long long)gridDim.x * blockDim.x) {
    const float gr = reduce1_ordered(a, i) * gs;
    float p = a.master[i], m = a.m[i], v = a.rule == 0 ? a.v[i] : 0.f;
    apply_rule(a, h, gr, p, m, v);
    a.master[i] = p; a.m[i] = m; if (a.rule == 0) a.v[i] = v;
    a.shadow[a.rank][i] = __float2bfloat16(p);
  }
  __threadfence_system();
  handshake(a, 1, epoch);
  retire(a);
}

// ------------------------------------------------------------------------------------------------ two passes
__device__ __forceinline__ float block_sum_ordered(float v) {
  // fixed-shape tree: the result depends only on the per-thread values, not on timing
  __shared__ float sh[DP_THREADS / 32];
  v = warp_sum(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = 0.f;
  if (threadIdx.x < 32) {
    t = threadIdx.x < DP_THREADS / 32 ? sh[threadIdx.x] : 0.f;
    t = warp_sum(t);
  }
  __shared__ float s_out;
  if (threadIdx.x == 0) s_out = t;
  __syncthreads();
  return s_out;
}

__device__ __forceinline__ int seg_of(const DpFusedArgs& a, long long i) {
  int s = a.blk_seg[i >> 10];
  while (s + 1 < a.nseg && i >= a.seg_off[2 * (s + 1)]) ++s;
  return s;
}

__global__ void __launch_bounds__(DP_THREADS, 1) dp_reduce_kernel(const __grid_constant__ DpFusedArgs a) {
  const uint32_t epoch = a.words[0] + 1u;
  if (!handshake(a, 0, epoch)) { retire(a); return; }
  const int par = a.words[2] & 1;
  const int table = a.nseg > 0 ? a.nseg : 1;
  float* my_partial = a.partial[a.rank] + (size_t)par * table;
  const float inv_w = a.red_scale;

  const long long shard = (a.end - a.begin) / a.world;
  const long long base = a.begin + shard * a.rank;
  const long long n8 = shard / 8;
  // contiguous span per CTA, so that a thread meets the tensors in ascending order and flushes rarely
  const long long per = (n8 + gridDim.x - 1) / gridDim.x;
  const long long lo = per * blockIdx.x, hi = min(n8, lo + per);
  int cur = -1; float acc = 0.f;
  for (long long i8 = lo + threadIdx.x; i8 < hi; i8 += blockDim.x) {
    const long long i = base + i8 * 8;
    float g[8];
    reduce8(a, i, g);
#pragma unroll
    for (int j = 0; j < 8; ++j) g[j] *= inv_w;
    *reinterpret_cast<float4*>(a.grad[a.rank] + i) = make_float4(g[0], g[1], g[2], g[3]);
    *reinterpret_cast<float4*>(a.grad[a.rank] + i + 4) = make_float4(g[4], g[5], g[6], g[7]);
    if (a.scale_mode == 2) {
      int s = seg_of(a, i);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        while (s + 1 < a.nseg && i + j >= a.seg_off[2 * (s + 1)]) ++s;     // packed tensors may meet inside a group of 8
        if (s != cur) { if (cur >= 0 && acc != 0.f) atomicAdd(my_partial + cur, acc); cur = s; acc = 0.f; }
        acc += g[j] * g[j];
      }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) acc += g[j] * g[j];
      cur = 0;
    }
  }
  if (a.scale_mode == 2) {
    if (cur >= 0 && acc != 0.f) atomicAdd(my_partial + cur, acc);
  } else {
    const float t = block_sum_ordered(acc);
    if (threadIdx.x == 0 && t != 0.f) atomicAdd(my_partial, t);
  }
  // replicated tensors: one CTA per tensor, everything in a fixed order => identical bits on every rank
  for (int s = a.first_rep_seg + blockIdx.x; s < a.nseg && a.rep_end > a.rep_begin; s += gridDim.x) {
    const long long sb = a.seg_off[2 * s], se = a.seg_off[2 * s + 1];
    float q = 0.f;
    for (long long i = sb + threadIdx.x; i < se; i += blockDim.x) {
      const float g = reduce1_ordered(a, i) * inv_w;
      a.red_rep[i - a.rep_begin] = g;
      q += g * g;
    }
    const float t = block_sum_ordered(q);
    if (threadIdx.x == 0) a.rep_sumsq[s] = t;
  }
  retire(a);
}

__global__ void __launch_bounds__(DP_THREADS, 1) dp_update_kernel(const __grid_constant__ DpFusedArgs a) {
  const uint32_t epoch = a.words[0] + 1u;
  if (!handshake(a, 0, epoch)) { retire(a); return; }      // every rank has finished its reduce pass
  const int par = a.words[2] & 1;
  const int table = a.nseg > 0 ? a.nseg : 1;
  const Hyper h = make_hyper(a);

  float coef = h.gs;                                          // scale_mode 1: one coefficient for everything
  if (a.scale_mode == 1) {
    float q = 0.f;
    for (int s = a.first_rep_seg + threadIdx.x; s < a.nseg; s += blockDim.x) q += a.rep_sumsq[s];
    float total = block_sum_ordered(q);
    for (int p = 0; p < a.world; ++p) total += ld_peer_f1(a.partial[p] + (size_t)par * table);
    const float norm = sqrtf(total);
    if (a.clip_max_norm > 0.f) coef *= fminf(1.f, a.clip_max_norm / (norm + 1e-6f));
    if (a.norm_out && blockIdx.x == 0 && threadIdx.x == 0) *a.norm_out = norm;
  }
  auto seg_scale = [&](int s) -> float {                      // scale_mode 2: 1 / max(rms of the tensor, eps)
    float total;
    if (s >= a.first_rep_seg) {
      total = a.rep_sumsq[s];
    } else {
      total = 0.f;
      for (int p = 0; p < a.world; ++p) total += ld_peer_f1(a.partial[p] + (size_t)par * table + s);
    }
    const long long numel = a.seg_off[2 * s + 1] - a.seg_off[2 * s];
    return h.gs / fmaxf(sqrtf(total / (float)(numel > 0 ? numel : 1)), a.eps);
  };

  const long long shard = (a.end - a.begin) / a.world;
  const long long base = a.begin + shard * a.rank;
  const long long n8 = shard / 8;
  const long long per = (n8 + gridDim.x - 1) / gridDim.x;
  const long long lo = per * blockIdx.x, hi = min(n8, lo + per);
  int cur = -1; float cur_scale = coef;
  for (long long i8 = lo + threadIdx.x; i8 < hi; i8 += blockDim.x) {
    const long long i = base + i8 * 8;
    float g[8];
    *reinterpret_cast<float4*>(g) = *reinterpret_cast<const float4*>(a.grad[a.rank] + i);
    *reinterpret_cast<float4*>(g + 4) = *reinterpret_cast<const float4*>(a.grad[a.rank] + i + 4);
    if (a.scale_mode == 2) {
      int s = seg_of(a, i);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        while (s + 1 < a.nseg && i + j >= a.seg_off[2 * (s + 1)]) ++s;
        if (s != cur) { cur = s; cur_scale = seg_scale(s); }
        g[j] *= cur_scale;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) g[j] *= coef;
    }
    publish8(a, i, update8(a, h, i, g));
  }
  for (int s = a.first_rep_seg + blockIdx.x; s < a.nseg && a.rep_end > a.rep_begin; s += gridDim.x) {
    const long long sb = a.seg_off[2 * s], se = a.seg_off[2 * s + 1];
    const float sc = a.scale_mode == 2 ? seg_scale(s) : coef;
    for (long long i = sb + threadIdx.x; i < se; i += blockDim.x) {
      const float gr = a.red_rep[i - a.rep_begin] * sc;
      float p = a.master[i], m = a.m[i], v = a.rule == 0 ? a.v[i] : 0.f;
      apply_rule(a, h, gr, p, m, v);
      a.master[i] = p; a.m[i] = m; if (a.rule == 0) a.v[i] = v;
      a.shadow[a.rank][i] = __float2bfloat16(p);
    }
  }
  // the table of the other parity was last read one step ago and is written next step: clear it now
  if (a.bump_pass) {
    float* other = a.partial[a.rank] + (size_t)(par ^ 1) * table;
    for (int s = blockIdx.x * blockDim.x + threadIdx.x; s < table; s += gridDim.x * blockDim.x) other[s] = 0.f;
  }
  __threadfence_system();
  handshake(a, 1, epoch);
  retire(a);
}

}  // namespace b200

// The argument block is passed by value (it holds the peer pointers). `grid` must be identical on
// all ranks and at most DP_MAX_CTAS (<= number of SMs so that every CTA is resident).
// pass: 0 = one-pass Adam, 1 = reduce pass, 2 = update pass.
extern "C" int b200_dp_fused_launch(const b200::DpFusedArgs* args, int pass, int grid, cudaStream_t st) {
  using namespace b200;
  if (args->world < 1 || args->world > DP_MAX_WORLD || grid < 1 || grid > DP_MAX_CTAS) return -1;
  if ((args->end - args->begin) % (8LL * args->world) != 0 || args->begin % 8 != 0) return -2;
  if (pass != 0 && (args->seg_off == nullptr || args->blk_seg == nullptr || args->nseg < 1)) return -3;
  if (pass == 0) dp_fused_adam_kernel<<<grid, DP_THREADS, 0, st>>>(*args);
  else if (pass == 1) dp_reduce_kernel<<<grid, DP_THREADS, 0, st>>>(*args);
  else if (pass == 2) dp_update_kernel<<<grid, DP_THREADS, 0, st>>>(*args);
  else return -4;
  return (int)cudaGetLastError();
}

extern "C" int b200_dp_flag_words() { return 2 * b200::DP_MAX_WORLD * b200::DP_MAX_CTAS; }
