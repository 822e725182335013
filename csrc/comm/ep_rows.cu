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
//   ep_push_counts  every rank stores its per-expert row counts into its slot of every peer's count table (double
//                 buffered by call parity); after the next barrier each rank knows all ranks' counts without a
//                 library collective.
//   ep_plan       routing plan in one pass: from the count table it derives, for every local (token, slot) entry,
//                 the destination rank and the row in that rank's expert-contiguous, 128-padded buffer (or -1 when
//                 the destination's capacity is exhausted: the row is dropped), the record that travels with the
//                 row, and this rank's own padded expert offsets, truncated at the capacity.
//   ep_resolve    turns the records an expert rank has received into byte addresses: where to fetch each row from
//                 (the sender's token buffer) and where to send its result back (the sender's receive buffer).
// The same kernels serve the backward pass (push of output gradients, pull of input gradients).
// Rows whose rank entry is negative are skipped (push) or zero-filled (pull).  Plain ld/st on peer-mapped
// addresses only; ordering against the consumer is provided by the symmetric barrier around the calls.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cstdint>
#include "../api.h"
#include "../common/bounds.cuh"

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

constexpr int kCountSlots = 512;  // experts per count-table row

__global__ void ep_push_counts_kernel(const int64_t* __restrict__ counts, PeerPtrs tables, int rank, int R, int E,
                                      int parity) {
  for (int i = threadIdx.x; i < R * E; i += blockDim.x) {
    const int peer = i / E, e = i % E;
    reinterpret_cast<int*>(tables.p[peer])[(parity * kMaxPeers + rank) * kCountSlots + e] = (int)counts[e];
  }
}

// table: this rank's copy, int[2][kMaxPeers][kCountSlots].  pos_l / off_l: padded local position of every entry and
// padded local offsets per expert from the local counting sort (their difference is the entry's stable rank inside
// its expert).
__global__ void ep_plan_kernel(const int64_t* __restrict__ flat, const int64_t* __restrict__ pos_l,
                               const int* __restrict__ off_l, const float* __restrict__ w,
                               const int* __restrict__ table, int rank, int R, int E, int El, int64_t cap, int K,
                               int64_t NK, int* __restrict__ dst_rank, int64_t* __restrict__ dst_pos,
                               int64_t* __restrict__ home_pos, int* __restrict__ off_local, int* __restrict__ tags,
                               unsigned long long* __restrict__ dropped) {
  __shared__ int64_t s_start[kCountSlots];  // first row, at its destination, of this rank's entries for expert e
  __shared__ int s_pad[kCountSlots];
  __shared__ int s_before[kCountSlots];
  __shared__ unsigned int s_drop;
  if (threadIdx.x == 0) s_drop = 0;
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int total = 0, before = 0;
    for (int r = 0; r < R; ++r) {
      const int c = table[r * kCountSlots + e];
      total += c;
      if (r < rank) before += c;
    }
    s_pad[e] = (total + 127) / 128 * 128;
    s_before[e] = before;
  }
  __syncthreads();
  for (int r = threadIdx.x; r < R; r += blockDim.x) {  // padded offsets inside every destination rank
    int64_t run = 0;
    for (int j = 0; j < El; ++j) {
      const int e = r * El + j;
      s_start[e] = run + s_before[e];
      if (r == rank && blockIdx.x == 0) off_local[j] = (int)(run < cap ? run : cap);
      run += s_pad[e];
    }
    if (r == rank && blockIdx.x == 0) off_local[El] = (int)(run < cap ? run : cap);
  }
  __syncthreads();
  unsigned int my_drop = 0;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < NK; i += (int64_t)gridDim.x * blockDim.x) {
    int e = (int)flat[i];
    const bool valid = MT_IN_BOUNDS(e, E);  // debug-bounds build: a bad expert id is reported and its row dropped
    if (!valid) e = 0;
    const int r = e / El;
    const int64_t pos = s_start[e] + (pos_l[i] - off_l[e]);
    const bool keep = valid && pos < cap;
    dst_rank[i] = keep ? r : -1;
    dst_pos[i] = keep ? pos : 0;
    home_pos[i] = keep ? i : -1;
    int4 t;
    t.x = rank + 1;
    t.y = (int)i;
    t.z = (int)(i / K);
    t.w = __float_as_int(w[i]);
    reinterpret_cast<int4*>(tags)[i] = t;
    my_drop += keep ? 0u : 1u;
  }
  if (my_drop) atomicAdd(&s_drop, my_drop);
  __syncthreads();
  if (threadIdx.x == 0 && s_drop) atomicAdd(dropped, (unsigned long long)s_drop);
}

__global__ void ep_resolve_kernel(const int* __restrict__ tags, PeerPtrs in_bufs, PeerPtrs out_bufs, int64_t cap,
                                  int64_t row_bytes, unsigned long long* __restrict__ row_src,
                                  unsigned long long* __restrict__ row_dst, float* __restrict__ scale) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < cap; i += (int64_t)gridDim.x * blockDim.x) {
    const int4 t = reinterpret_cast<const int4*>(tags)[i];
    unsigned long long src = 0, dst = 0;
    if (t.x > 0 && t.x <= kMaxPeers) {
      src = reinterpret_cast<unsigned long long>(in_bufs.p[t.x - 1]) + (unsigned long long)t.z * row_bytes;
      dst = reinterpret_cast<unsigned long long>(out_bufs.p[t.x - 1]) + (unsigned long long)t.y * row_bytes;
    }
    row_src[i] = src;
    row_dst[i] = dst;
    scale[i] = __int_as_float(t.w);
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

int ep_count_slots() { return kCountSlots; }

void ep_push_counts(const int64_t* counts, const PeerPtrs& tables, int rank, int R, int E, int parity,
                    cudaStream_t stream) {
  ep_push_counts_kernel<<<1, 256, 0, stream>>>(counts, tables, rank, R, E, parity);
}

void ep_plan(const int64_t* flat, const int64_t* pos_l, const int* off_l, const float* w, const int* table, int rank, int R,
             int E, int El, int64_t cap, int K, int64_t NK, int* dst_rank, int64_t* dst_pos, int64_t* home_pos,
             int* off_local, int* tags, unsigned long long* dropped, cudaStream_t stream) {
  if (NK <= 0) return;
  ep_plan_kernel<<<grid_for(NK), 256, 0, stream>>>(flat, pos_l, off_l, w, table, rank, R, E, El, cap, K, NK, dst_rank,
                                                   dst_pos, home_pos, off_local, tags, dropped);
}

void ep_resolve(const int* tags, const PeerPtrs& in_bufs, const PeerPtrs& out_bufs, int64_t cap, int64_t row_bytes,
                unsigned long long* row_src, unsigned long long* row_dst, float* scale, cudaStream_t stream) {
  if (cap <= 0) return;
  ep_resolve_kernel<<<grid_for(cap), 256, 0, stream>>>(tags, in_bufs, out_bufs, cap, row_bytes, row_src, row_dst, scale);
}

void ep_gather_rows(void* out, const unsigned long long* row_src, const float* row_scale, int64_t rows, int dim,
                    cudaStream_t stream) {
  if (rows == 0) return;
  ep_gather_rows_kernel<<<grid_for(rows * (dim / 8)), 256, 0, stream>>>((__nv_bfloat16*)out, row_src, row_scale, rows, dim);
}

}  // namespace mt
