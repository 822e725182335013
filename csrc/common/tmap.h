// Host-side helpers: TMA tensor-map encoding through the driver entry point (no link-time
// dependency on libcuda), status words, error checks.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdint>
#include <stdexcept>
#include <string>

namespace mt {

#define MT_CUDA_CHECK(expr)                                                                          \
  do {                                                                                               \
    cudaError_t _e = (expr);                                                                         \
    if (_e != cudaSuccess)                                                                           \
      throw std::runtime_error(std::string(#expr) + " failed: " + cudaGetErrorString(_e));          \
  } while (0)

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn get_encode_tiled() {
  // The encoder is a driver-API call and needs a context current in the calling thread.  A thread that has only
  // ever been handed cached device memory (an autograd worker whose first operation is one of these GEMMs) has
  // none yet: the runtime binds the primary context lazily on its first runtime call, so make one here.
  thread_local bool context_bound = false;
  if (!context_bound) {
    MT_CUDA_CHECK(cudaFree(nullptr));
    context_bound = true;
  }
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    MT_CUDA_CHECK(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q));
    if (q != cudaDriverEntryPointSuccess || !p) throw std::runtime_error("cuTensorMapEncodeTiled unavailable");
    fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// 2-D row-major tensor [rows, cols] with `ld` elements between rows; box = [box_rows, box_cols].
// The TMA rules checked here: 16-byte aligned base, row pitch a multiple of 16 bytes, inner box
// extent a multiple of 16 bytes and (for swizzled modes) no wider than the swizzle span.
inline CUtensorMap make_tmap_2d(const void* base, CUtensorMapDataType dt, int elem_bytes, uint64_t rows,
                                uint64_t cols, uint64_t ld, uint32_t box_rows, uint32_t box_cols,
                                CUtensorMapSwizzle swz) {
  if (reinterpret_cast<uintptr_t>(base) % 16 != 0) throw std::runtime_error("TMA base must be 16-byte aligned");
  if ((ld * elem_bytes) % 16 != 0) throw std::runtime_error("TMA row pitch must be a multiple of 16 bytes");
  if ((box_cols * elem_bytes) % 16 != 0) throw std::runtime_error("TMA inner box must be a multiple of 16 bytes");
  if (box_rows > 256 || box_cols > 256) throw std::runtime_error("TMA box dims must be <= 256");
  CUtensorMap m;
  cuuint64_t gdim[2] = {cols, rows};
  cuuint64_t gstride[1] = {ld * static_cast<uint64_t>(elem_bytes)};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = get_encode_tiled()(&m, dt, 2, const_cast<void*>(base), gdim, gstride, box, estr,
                                  CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) throw std::runtime_error("cuTensorMapEncodeTiled failed: " + std::to_string((int)r));
  return m;
}

// 3-D tensor [d2, d1, d0] (d0 innermost) with strides (in elements) s2, s1 and unit inner stride.
inline CUtensorMap make_tmap_3d(const void* base, CUtensorMapDataType dt, int elem_bytes, uint64_t d2, uint64_t d1,
                                uint64_t d0, uint64_t s2, uint64_t s1, uint32_t b2, uint32_t b1, uint32_t b0,
                                CUtensorMapSwizzle swz) {
  if (reinterpret_cast<uintptr_t>(base) % 16 != 0) throw std::runtime_error("TMA base must be 16-byte aligned");
  if ((s1 * elem_bytes) % 16 != 0 || (s2 * elem_bytes) % 16 != 0)
    throw std::runtime_error("TMA strides must be multiples of 16 bytes");
  if ((b0 * elem_bytes) % 16 != 0) throw std::runtime_error("TMA inner box must be a multiple of 16 bytes");
  CUtensorMap m;
  cuuint64_t gdim[3] = {d0, d1, d2};
  cuuint64_t gstride[2] = {s1 * static_cast<uint64_t>(elem_bytes), s2 * static_cast<uint64_t>(elem_bytes)};
  cuuint32_t box[3] = {b0, b1, b2};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = get_encode_tiled()(&m, dt, 3, const_cast<void*>(base), gdim, gstride, box, estr,
                                  CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) throw std::runtime_error("cuTensorMapEncodeTiled(3d) failed: " + std::to_string((int)r));
  return m;
}

}  // namespace mt
