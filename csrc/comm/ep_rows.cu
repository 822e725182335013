// Expert-parallel token exchange over NVLink peer memory (one process per GPU, buffers in symmetric memory).
//
//   ep_push_rows  dispatch: row r of a local [R, D] bf16 matrix is stored to row dst_pos[r] of the buffer of rank
//                 dst_rank[r] (its expert-contiguous, 128-padded input buffer).  Writing straight to the final
//                 position on the owning GPU fuses the routing permute with the all-to-all.
//   ep_pull_rows  combine: out[r] = buffer of rank src_rank[r], row src_pos[r] (the expert outputs stay where the
//                 grouped GEMM wrote them; the token's home rank pulls its K rows and reduces them locally).
//   ep_gather_rows  table-driven pull: out[r] = scale[r] * (the dim-wide bf16 row at byte address row_src[r]), or a zero
//                 row where the address is 0.  The addresses point into peers' (or this rank's) symmetric buffers, so
//                 one pass both fetches the rows over NVLink and lays them out expert-contiguous and padded; with
//                 per-row scales it also applies the routing weight of the combine's backward on the fly.
// The same kernels serve the backward pass (push of output gradients, pull of input gradients).
// Rows whose rank entry is negative are skipped (push) or zero-filled (pull).  Plain ld/st on peer-mapped
// addresses only; ordering against the consumer is provided by the symmetric barrier around the calls.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cstdint>
#include "../api.h"

namespace mt {
namespace {

__global__ void ep_push_rows_kernel(const __nv_bfloat16* __restrict__ src, const int* __restrict__ dst_rank,
                                    const int64_t* __restrict__ dst_pos, PeerPtrs bufs, int64_t rows, int dim,
                                    int64_t cap_rows, int* overflow) {
  const int nvec = dim >> 3;
  const int64_t total = rows * nvec;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = idx / nvec;
    const int c = (int)(idx % nvec);
    const int rk = dst_rank[r];
    if (rk < 0) continue;
    const int64_t pos = dst_pos[r];
    if (pos < 0 || pos >= cap_rows) {  // receiver's buffer is full: record it, never write out of bounds
      if (c == 0 && overflow) atomicExch(overflow, 1);
      continue;
    }
    const uint4 v = reinterpret_cast<const uint4*>(src + r * dim)[c];
    reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(bufs.p[rk]) + pos * dim)[c] = v;
  }
}

__global__ void ep_pull_rows_kernel(__nv_bfloat16* __restrict__ out, const int* __restrict__ src_rank,
                                    const int64_t* __restrict__ src_pos, PeerPtrs bufs, int64_t rows, int dim,
                                    int64_t cap_rows) {
  const int nvec = dim >> 3;
  const int64_t total = rows * nvec;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = idx / nvec;
    const int c = (int)(idx % nvec);
    const int rk = src_rank[r];
    const int64_t pos = src_pos[r];
    uint4 v = make_uint4(0, 0, 0, 0);
    if (rk >= 0 && pos >= 0 && pos < cap_rows)
      v = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(bufs.p[rk]) + pos * dim)[c];
    reinterpret_cast<uint4*>(out + r * dim)[c] = v;
  }
}

__global__ void ep_gather_rows_kernel(__nv_bfloat16* __restrict__ out, const unsigned long long* __restrict__ row_src,
                                      const float* __restrict__ row_scale, int64_t rows, int dim) {
  const int nvec = dim >> 3;
  const int64_t total = rows * nvec;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = idx / nvec;
    const int c = (int)(idx % nvec);
    const unsigned long long src = row_src[r];
    uint4 v = make_uint4(0, 0, 0, 0);
    if (src != 0) {
      v = reinterpret_cast<const uint4*>(src)[c];
      if (row_scale != nullptr) {
        const float sc = row_scale[r];
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __bfloat1622float2(h[j]);
          h[j] = __floats2bfloat162_rn(f.x * sc, f.y * sc);
        }
      }
    }
    reinterpret_cast<uint4*>(out + r * dim)[c] = v;
  }
}

inline int grid_for(int64_t total) {
  int64_t b = (total + 255) / 256;
  return (int)(b > 148 * 16 ? 148 * 16 : (b < 1 ? 1 : b));
}

}  // namespace

void ep_push_rows(const void* src, const int* dst_rank, const int64_t* dst_pos, const PeerPtrs& bufs, int64_t rows,
                  int dim, int64_t cap_rows, int* overflow, cudaStream_t stream) {
  if (rows == 0) return;
  ep_push_rows_kernel<<<grid_for(rows * (dim / 8)), 256, 0, stream>>>((const __nv_bfloat16*)src, dst_rank, dst_pos, bufs,
                                                                    rows, dim, cap_rows, overflow);
}

void ep_pull_rows(void* out, const int* src_rank, const int64_t* src_pos, const PeerPtrs& bufs, int64_t rows, int dim,
                  int64_t cap_rows, cudaStream_t stream) {
  if (rows == 0) return;
  ep_pull_rows_kernel<<<grid_for(rows * (dim / 8)), 256, 0, stream>>>((__nv_bfloat16*)out, src_rank, src_pos, bufs, rows,
                                                                    dim, cap_rows);
}

void ep_gather_rows(void* out, const unsigned long long* row_src, const float* row_scale, int64_t rows, int dim,
                    cudaStream_t stream) {
  if (rows == 0) return;
  ep_gather_rows_kernel<<<grid_for(rows * (dim / 8)), 256, 0, stream>>>((__nv_bfloat16*)out, row_src, row_scale, rows, dim);
}

}  // namespace mt
