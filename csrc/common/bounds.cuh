// Checked indexing for the debug-bounds build (-DMINTEXT_DEBUG_BOUNDS).
//
// Kernels that index memory with values they READ from memory (token ids, targets, positions, expert ids, row
// tables) wrap the value in MT_IN_BOUNDS(index, limit).  In the ordinary build the macro is the constant `true` and
// costs nothing.  In the debug-bounds build it tests 0 <= index < limit; the first violation of a translation unit
// is recorded (source line, offending index, limit) in a per-unit device record and the macro yields false, so that
// the kernel skips the access instead of faulting.  The host collects the records through
// mt::debug_bounds_report() (bindings: debug_bounds_report / debug_bounds_reset).  This is the in-tree stand-in for
// an external memory checker: a bad index becomes a report the host can read, and the context stays usable.
//
// One record per translation unit (a file-scope __device__ variable): no relocatable device code is needed.
// Include this header in a .cu file after <cuda_runtime.h>.
#pragma once
#include <cuda_runtime.h>

namespace mt {
struct BoundsRecord {
  int code;          // 0 = clean, 1 = a violation was recorded
  int line;          // source line of the MT_IN_BOUNDS that failed
  long long index;   // offending value
  long long limit;   // exclusive upper bound it was tested against
};
using BoundsReadFn = int (*)(BoundsRecord*);
using BoundsResetFn = void (*)();
// host registry (bindings.cpp): every translation unit built with the flag registers its reader at load time
void register_bounds_unit(const char* file, BoundsReadFn read, BoundsResetFn reset);
}  // namespace mt

#if defined(MINTEXT_DEBUG_BOUNDS) && defined(__CUDACC__)  // device code: only in files nvcc compiles
namespace {
__device__ mt::BoundsRecord g_mt_bounds;

__device__ __forceinline__ bool mt_in_bounds(long long i, long long n, int line) {
  if (i >= 0 && i < n) return true;
  if (atomicCAS(&g_mt_bounds.code, 0, 1) == 0) {
    g_mt_bounds.line = line;
    g_mt_bounds.index = i;
    g_mt_bounds.limit = n;
  }
  return false;
}

int mt_bounds_read(mt::BoundsRecord* out) {
  return static_cast<int>(cudaMemcpyFromSymbol(out, g_mt_bounds, sizeof(mt::BoundsRecord)));
}
void mt_bounds_reset() {
  const mt::BoundsRecord zero{0, 0, 0, 0};
  cudaMemcpyToSymbol(g_mt_bounds, &zero, sizeof(zero));
}
struct MtBoundsRegistrar {
  MtBoundsRegistrar() { mt::register_bounds_unit(__BASE_FILE__, &mt_bounds_read, &mt_bounds_reset); }  // the .cu file
};
static MtBoundsRegistrar g_mt_bounds_registrar;
}  // namespace
#define MT_IN_BOUNDS(i, n) mt_in_bounds(static_cast<long long>(i), static_cast<long long>(n), __LINE__)
#else
#define MT_IN_BOUNDS(i, n) true
#endif
