// Host-side construction of TMA tensor maps. The driver entry point is resolved at run time
// through the CUDA runtime, so the library links against cudart only and can be imported on a
// machine without a driver (nothing here runs until the first launch).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdint>
#include <cstdio>
#include <mutex>

namespace b200 {

typedef CUresult (*PFN_encodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                    CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                    CUtensorMapFloatOOBfill);

inline PFN_encodeTiled get_encode_fn() {
  static PFN_encodeTiled fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<PFN_encodeTiled>(p);
    }
  });
  return fn;
}

// cuTensorMapEncodeTiled is a driver call and needs a current context on the calling thread. A fresh
// thread (e.g. an autograd worker) that has made no runtime call yet has none, so bind the primary
// context of the runtime's current device once per thread.
inline void ensure_context() {
  thread_local bool bound = false;
  if (!bound) {
    int d = 0;
    if (cudaGetDevice(&d) == cudaSuccess) cudaSetDevice(d);
    bound = true;
  }
}

// 3-D map over a row-major [batch][rows][cols] view. `row_stride_bytes` and `batch_stride_bytes`
// must be multiples of 16; `base` must be 16-byte aligned. Box = {box_cols, box_rows, 1}.
// Returns 0 on success, a CUresult-like non-zero code otherwise.
inline int make_tmap_3d(CUtensorMap* out, const void* base, CUtensorMapDataType dt, uint32_t elem_bytes,
                        uint64_t cols, uint64_t rows, uint64_t batch, uint64_t row_stride_bytes,
                        uint64_t batch_stride_bytes, uint32_t box_cols, uint32_t box_rows,
                        CUtensorMapSwizzle swz) {
  ensure_context();
  PFN_encodeTiled fn = get_encode_fn();
  if (!fn) return -1;
  cuuint64_t gdim[3] = {cols, rows, batch};
  cuuint64_t gstr[2] = {row_stride_bytes, batch > 1 ? batch_stride_bytes : row_stride_bytes * rows};
  if (gstr[1] % 16 != 0) gstr[1] = (gstr[1] + 15) / 16 * 16;
  cuuint32_t box[3] = {box_cols, box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  (void)elem_bytes;
  CUresult r = fn(out, dt, 3, const_cast<void*>(base), gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return static_cast<int>(r);
}

// 4-D map for attention operands: element (b, s, h, e) lives at base + b*sb + s*ss + h*sh + e
// (strides in elements, e contiguous). Dimensions are ordered {e, h, s, b}; the box is
// {box_e, 1, box_s, 1}, so a tile lands in shared memory as [box_s rows][box_e] (rows of 128 bytes
// when box_e * elem = 128). All byte strides must be multiples of 16.
inline int make_tmap_attn(CUtensorMap* out, const void* base, CUtensorMapDataType dt, uint32_t elem_bytes,
                          uint64_t hd, uint64_t H, uint64_t S, uint64_t B, uint64_t sh, uint64_t ss, uint64_t sb,
                          uint32_t box_e, uint32_t box_s, CUtensorMapSwizzle swz) {
  ensure_context();
  PFN_encodeTiled fn = get_encode_fn();
  if (!fn) return -1;
  cuuint64_t gdim[4] = {hd, H, S, B};
  cuuint64_t gstr[3] = {sh * elem_bytes, ss * elem_bytes, sb * elem_bytes};
  cuuint32_t box[4] = {box_e, 1, box_s, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(out, dt, 4, const_cast<void*>(base), gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return static_cast<int>(r);
}

}  // namespace b200
