// Token-embedding gather (bf16 table -> bf16 rows, optional scale) and its backward: a scatter-add of the
// output gradient rows into an fp32 table gradient (atomics; duplicate ids are summed).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cstdint>
#include "../api.h"
#include "../common/bounds.cuh"

namespace mt {
namespace {

union Pack8 {
  uint4 u;
  __nv_bfloat16 h[8];
};

__global__ void embedding_fwd_kernel(const __nv_bfloat16* __restrict__ table, const int64_t* __restrict__ ids,
                                     __nv_bfloat16* __restrict__ out, int64_t tokens, int dim, float scale,
                                     int use_scale, int64_t vocab) {
  const int nvec = dim >> 3;
  const int64_t total = tokens * nvec;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t t = idx / nvec;
    const int c = (int)(idx % nvec);
    Pack8 a;
    if (!MT_IN_BOUNDS(ids[t], vocab)) continue;  // debug-bounds build: a bad token id is reported, not dereferenced
    a.u = reinterpret_cast<const uint4*>(table + ids[t] * dim)[c];
    if (use_scale) {
      const __nv_bfloat16 s = __float2bfloat16(scale);
#pragma unroll
      for (int j = 0; j < 8; ++j) a.h[j] = __hmul(a.h[j], s);
    }
    reinterpret_cast<uint4*>(out + t * dim)[c] = a.u;
  }
}

__global__ void embedding_bwd_kernel(const __nv_bfloat16* __restrict__ dout, const int64_t* __restrict__ ids,
                                     float* __restrict__ dtable, int64_t tokens, int dim, float scale, int64_t vocab) {
  const int nvec = dim >> 3;
  const int64_t total = tokens * nvec;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t t = idx / nvec;
    const int c = (int)(idx % nvec);
    Pack8 a;
    a.u = reinterpret_cast<const uint4*>(dout + t * dim)[c];
    if (!MT_IN_BOUNDS(ids[t], vocab)) continue;
    float* dst = dtable + ids[t] * dim + c * 8;
#pragma unroll
    for (int j = 0; j < 8; ++j) atomicAdd(dst + j, __bfloat162float(a.h[j]) * scale);
  }
}

inline int grid_for(int64_t total) {
  int64_t b = (total + 255) / 256;
  return (int)(b > 148 * 32 ? 148 * 32 : b);
}

}  // namespace

void embedding_fwd(const void* table, const int64_t* ids, void* out, int64_t tokens, int dim, float scale,
                   int64_t vocab, cudaStream_t stream) {
  const int64_t total = tokens * (dim / 8);
  if (total == 0) return;
  embedding_fwd_kernel<<<grid_for(total), 256, 0, stream>>>((const __nv_bfloat16*)table, ids, (__nv_bfloat16*)out,
                                                           tokens, dim, scale, scale != 1.0f, vocab);
}

void embedding_bwd(const void* dout, const int64_t* ids, float* dtable, int64_t tokens, int dim, float scale,
                   int64_t vocab, cudaStream_t stream) {
  const int64_t total = tokens * (dim / 8);
  if (total == 0) return;
  embedding_bwd_kernel<<<grid_for(total), 256, 0, stream>>>((const __nv_bfloat16*)dout, ids, dtable, tokens, dim,
                                                           scale, vocab);
}

}  // namespace mt
