// Host-side construction of TMA tensor maps without linking libcuda: the encoder is looked up
// through the runtime's driver entry-point query.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

namespace yv {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn get_encode_tiled() {
  // The encoder is a driver call and fails (invalid context) in a thread that has not yet made a runtime call of
  // its own, e.g. a fresh autograd worker whose first device work is a TMA kernel.  A null free is the cheapest
  // runtime call that binds the device's primary context to the calling thread.
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) {
    cudaFree(nullptr);
    ctx_bound = true;
  }
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || p == nullptr) {
      fprintf(stderr, "pisceslx_b200: cuTensorMapEncodeTiled unavailable (%d)\n", static_cast<int>(e));
      return nullptr;
    }
    fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// 2-D row-major tensor [outer, inner] with row pitch `ld_elems`; box = [box_outer, box_inner];
// 128-byte swizzle (box_inner * elem_bytes must be 128).  Returns 0 on success.
inline int make_tmap_2d(CUtensorMap* map, CUtensorMapDataType dt, int elem_bytes, const void* base, uint64_t inner,
                        uint64_t outer, uint64_t ld_elems, uint32_t box_inner, uint32_t box_outer,
                        CUtensorMapSwizzle swz = CU_TENSOR_MAP_SWIZZLE_128B) {
  EncodeTiledFn fn = get_encode_tiled();
  if (fn == nullptr) return -1;
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0 || ((ld_elems * elem_bytes) & 15u) != 0) return -2;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {ld_elems * static_cast<uint64_t>(elem_bytes)};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -3;
}

// 3-D tensor [d2, d1, d0(inner)] with byte strides s1 (d1) and s2 (d2).
inline int make_tmap_3d(CUtensorMap* map, CUtensorMapDataType dt, int elem_bytes, const void* base, uint64_t d0,
                        uint64_t d1, uint64_t d2, uint64_t s1_bytes, uint64_t s2_bytes, uint32_t b0, uint32_t b1,
                        uint32_t b2, CUtensorMapSwizzle swz = CU_TENSOR_MAP_SWIZZLE_128B) {
  EncodeTiledFn fn = get_encode_tiled();
  if (fn == nullptr) return -1;
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0 || (s1_bytes & 15u) != 0 || (s2_bytes & 15u) != 0) return -2;
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {s1_bytes, s2_bytes};
  cuuint32_t box[3] = {b0, b1, b2};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, dt, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  (void)elem_bytes;
  return r == CUDA_SUCCESS ? 0 : -3;
}

}  // namespace yv
