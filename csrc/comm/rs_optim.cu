// Sharded optimizer step over NVLink peer memory (one process per GPU, buffers in symmetric memory).
//
//   symm_barrier        every rank posts a sequence number into each peer's flag slot and waits (bounded) until all
//                       peers' numbers have arrived in its own slots.
//   grad_pull_reduce    reduce-scatter by pulling: this rank reads its shard range from every rank's flat fp32
//                       gradient buffer with plain peer loads (its own copy included), sums in a fixed rank order,
//                       keeps the sum locally and accumulates its sum of squares for the global-norm clip.
//   grad_pull_bucket    the same reduction for one bucket of the flat buffer, launched on a side stream while the
//                       backward pass is still running: the kernel first posts "my gradients for bucket b are
//                       final" (a sequence number) into every peer's flag table, waits (bounded) until every peer
//                       has posted the same, then pulls and sums its slice of the bucket from all ranks and
//                       stores zeros back into the slices it has consumed (`clear`), so that no separate clearing pass
//                       over the gradient buffers is needed.  Those are remote stores: a rank may write the cleared
//                       range again only after a later synchronisation point that is far behind them (the step-end
//                       barrier); a caller that reuses the buffer right away passes clear = false and clears its own
//                       memory once every peer has finished reading.  Runs on a capped grid so that it hides under the backward
//                       kernels instead of competing with them.
//   adamw_publish       fused AdamW on the shard (clip factor, moments, fp32 master) whose bf16 result is written
//                       straight into the shard's slot of every rank's resident parameter buffer (peer stores),
//                       i.e. the update and the parameter all-gather are one kernel.
//   peer_gather         parameter all-gather for the parameter-sharded engine mode: every rank keeps only its 1/N slice
//                       of a layer's bf16 weights; before the layer runs, this kernel copies slice r from rank r's
//                       shard buffer (plain 16-byte peer loads) into the local staging buffer, one layer ahead of
//                       the compute stream.
// No multimem / multicast is used here; all remote traffic is ordinary ld/st on peer-mapped addresses.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cstdint>
#include "../api.h"
#include "../common/ptx.cuh"

namespace mt {
namespace {

__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// flags: per rank an int[kMaxPeers] array in symmetric memory; slot r of rank d = last sequence number rank r posted.
__global__ void symm_barrier_kernel(PeerPtrs flags, int rank, int world, int seq, int* status) {
  const int peer = threadIdx.x;
  if (peer >= world) return;
  __threadfence_system();
  st_release_sys(reinterpret_cast<int*>(flags.p[peer]) + rank, seq);
  const int* mine = reinterpret_cast<const int*>(flags.p[rank]) + peer;
  const long long t0 = clock64();
  while (ld_acquire_sys(mine) < seq) {
    if (clock64() - t0 > kMaxWaitCycles) {
      if (status) atomicCAS(status, 0, MT_ERR_TIMEOUT_FLAG);
      return;
    }
  }
}

__global__ void grad_pull_reduce_kernel(PeerPtrs grads, int rank, int world, int64_t lo, int64_t n, float* out,
                                        float* sumsq) {
  const int64_t nvec = n >> 2;
  float acc = 0.f;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (int64_t)gridDim.x * blockDim.x) {
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
    // fixed summation order (rank 0 .. world-1) keeps the result identical on every run; the loads of the
    // different peers are independent and overlap in flight
#pragma unroll 8
    for (int r = 0; r < world; ++r) {
      const float4 v = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(grads.p[r]) + lo)[i];
      s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
    }
    reinterpret_cast<float4*>(out)[i] = s;
    acc += s.x * s.x + s.y * s.y + s.z * s.z + s.w * s.w;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  __shared__ float red[32];
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    acc = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (threadIdx.x == 0) atomicAdd(sumsq, acc);
  }
}

// The readiness handshake of one bucket on its own: posts this rank's sequence number to every peer and waits (bounded)
// for theirs.  One warp: while it waits it holds no shared memory and next to no registers, so it never keeps a compute
// kernel's blocks off an SM, which a waiting multi-block reduction grid does.
__global__ void bucket_ready_kernel(PeerPtrs flags, int rank, int world, int bucket, int seq, int* status) {
  const int peer = threadIdx.x;
  if (peer >= world) return;
  __threadfence_system();  // this rank's gradient writes (earlier kernels of the stream) before the post
  st_release_sys(reinterpret_cast<int*>(flags.p[peer]) + rank * kBucketSlots + bucket, seq);
  const int* mine = reinterpret_cast<const int*>(flags.p[rank]) + peer * kBucketSlots + bucket;
  const long long t0 = clock64();
  while (ld_acquire_sys(mine) < seq) {
    if (clock64() - t0 > kMaxWaitCycles) {
      if (status) atomicCAS(status, 0, MT_ERR_TIMEOUT_FLAG);
      return;
    }
  }
}

// flags: per rank an int[world * kBucketSlots] table in symmetric memory; entry [src * kBucketSlots + bucket] of rank d
// is the last sequence number rank src posted for that bucket.
__global__ void grad_pull_bucket_kernel(PeerPtrs grads, PeerPtrs flags, int rank, int world, int bucket, int seq,
                                        int64_t lo, int64_t n, float* __restrict__ out, int accumulate, int clear,
                                        int handshake, int* status) {
  __shared__ int give_up;
  // without the handshake a bucket_ready_kernel ran before this one on the same stream; if its wait expired the
  // status word is set and nothing may be read
  if (threadIdx.x == 0) give_up = (!handshake && status != nullptr && *reinterpret_cast<volatile int*>(status) != 0) ? 1 : 0;
  __syncthreads();
  if (handshake && threadIdx.x < world) {
    const int peer = threadIdx.x;
    if (blockIdx.x == 0) {
      __threadfence_system();  // this rank's gradient writes (earlier kernels of the stream) before the post
      st_release_sys(reinterpret_cast<int*>(flags.p[peer]) + rank * kBucketSlots + bucket, seq);
    }
    const int* mine = reinterpret_cast<const int*>(flags.p[rank]) + peer * kBucketSlots + bucket;
    const long long t0 = clock64();
    while (ld_acquire_sys(mine) < seq) {
      if (clock64() - t0 > kMaxWaitCycles) {
        if (status) atomicCAS(status, 0, MT_ERR_TIMEOUT_FLAG);
        give_up = 1;
        break;
      }
    }
  }
  __syncthreads();
  if (give_up) return;  // nothing is read or cleared: the host sees the status word
  const int64_t nvec = n >> 2;
  const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (int64_t)gridDim.x * blockDim.x) {
    // all peers' loads are issued before any of them is consumed or cleared, so they overlap in flight (a store
    // between two loads would pin their order: the buffers may alias as far as the compiler can tell)
    float4 v[kMaxPeers];
#pragma unroll
    for (int r = 0; r < kMaxPeers; ++r)
      if (r < world) v[r] = *(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(grads.p[r]) + lo) + i);
    float4 s = accumulate ? reinterpret_cast<const float4*>(out)[i] : zero;
#pragma unroll
    for (int r = 0; r < kMaxPeers; ++r)  // fixed summation order: the result is the same on every run
      if (r < world) { s.x += v[r].x; s.y += v[r].y; s.z += v[r].z; s.w += v[r].w; }
    reinterpret_cast<float4*>(out)[i] = s;
    if (clear) {
#pragma unroll
      for (int r = 0; r < kMaxPeers; ++r)  // this thread is the only reader of these elements: clear them for the next step
        if (r < world) *(reinterpret_cast<float4*>(reinterpret_cast<float*>(grads.p[r]) + lo) + i) = zero;
    }
  }
}

__global__ void adamw_publish_kernel(float* __restrict__ master, float* __restrict__ m, float* __restrict__ v,
                                     const float* __restrict__ grad, PeerPtrs params, int world, int64_t lo, int64_t n,
                                     float lr, float b1, float b2, float eps, float wd, float bc1, float bc2,
                                     float grad_scale, const float* __restrict__ clip_coef) {
  const float gs = clip_coef ? grad_scale * (*clip_coef) : grad_scale;
  const float rbc1 = __fdiv_rn(1.f, bc1), rbc2 = __fdiv_rn(1.f, bc2);  // IEEE-rounded, as in optim/adamw.cu
  const int64_t nvec = n >> 3;  // 8 elements = one 16-byte bf16 store per peer
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (int64_t)gridDim.x * blockDim.x) {
    float g[8], mm[8], vv[8], pp[8];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const float4 a = reinterpret_cast<const float4*>(grad)[2 * i + h];
      const float4 b = reinterpret_cast<const float4*>(m)[2 * i + h];
      const float4 c = reinterpret_cast<const float4*>(v)[2 * i + h];
      const float4 d = reinterpret_cast<const float4*>(master)[2 * i + h];
      g[4 * h] = a.x; g[4 * h + 1] = a.y; g[4 * h + 2] = a.z; g[4 * h + 3] = a.w;
      mm[4 * h] = b.x; mm[4 * h + 1] = b.y; mm[4 * h + 2] = b.z; mm[4 * h + 3] = b.w;
      vv[4 * h] = c.x; vv[4 * h + 1] = c.y; vv[4 * h + 2] = c.z; vv[4 * h + 3] = c.w;
      pp[4 * h] = d.x; pp[4 * h + 1] = d.y; pp[4 * h + 2] = d.z; pp[4 * h + 3] = d.w;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float gj = g[j] * gs;
      mm[j] = b1 * mm[j] + (1.f - b1) * gj;
      vv[j] = b2 * vv[j] + (1.f - b2) * gj * gj;
      pp[j] -= lr * (__fdiv_rn(mm[j] * rbc1, __fsqrt_rn(vv[j] * rbc2) + eps) + wd * pp[j]);
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      reinterpret_cast<float4*>(m)[2 * i + h] = make_float4(mm[4 * h], mm[4 * h + 1], mm[4 * h + 2], mm[4 * h + 3]);
      reinterpret_cast<float4*>(v)[2 * i + h] = make_float4(vv[4 * h], vv[4 * h + 1], vv[4 * h + 2], vv[4 * h + 3]);
      reinterpret_cast<float4*>(master)[2 * i + h] = make_float4(pp[4 * h], pp[4 * h + 1], pp[4 * h + 2], pp[4 * h + 3]);
    }
    uint4 o;
    o.x = pack_bf16x2(pp[0], pp[1]);
    o.y = pack_bf16x2(pp[2], pp[3]);
    o.z = pack_bf16x2(pp[4], pp[5]);
    o.w = pack_bf16x2(pp[6], pp[7]);
#pragma unroll 8
    for (int r = 0; r < world; ++r)
      reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(params.p[r]) + lo)[i] = o;
  }
}

// dst[r * n16 + i] = shards[r][lo16 + r * stride16 + i] in 16-byte units; the loads of all ranks are issued before
// the stores
__global__ void peer_gather_kernel(PeerPtrs shards, int world, int64_t lo16, int64_t stride16, int64_t n16,
                                   uint4* __restrict__ dst) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += (int64_t)gridDim.x * blockDim.x) {
    uint4 v[kMaxPeers];
#pragma unroll
    for (int r = 0; r < kMaxPeers; ++r)
      if (r < world) v[r] = *(reinterpret_cast<const uint4*>(shards.p[r]) + lo16 + r * stride16 + i);
#pragma unroll
    for (int r = 0; r < kMaxPeers; ++r)
      if (r < world) dst[(int64_t)r * n16 + i] = v[r];
  }
}

}  // namespace

void symm_barrier(const PeerPtrs& flags, int rank, int world, int seq, int* status, cudaStream_t stream) {
  symm_barrier_kernel<<<1, 32, 0, stream>>>(flags, rank, world, seq, status);
}

void peer_gather(const PeerPtrs& shards, int world, int64_t lo_bytes, int64_t rank_stride_bytes, int64_t n_bytes, void* dst,
                 int blocks, cudaStream_t stream) {
  if (n_bytes == 0) return;
  if (blocks <= 0) blocks = 64;
  peer_gather_kernel<<<blocks, 512, 0, stream>>>(shards, world, lo_bytes / 16, rank_stride_bytes / 16, n_bytes / 16,
                                                 reinterpret_cast<uint4*>(dst));
}

void grad_pull_reduce(const PeerPtrs& grads, int rank, int world, int64_t lo, int64_t n, float* out, float* sumsq,
                      cudaStream_t stream) {
  if (n == 0) return;
  grad_pull_reduce_kernel<<<148 * 8, 256, 0, stream>>>(grads, rank, world, lo, n, out, sumsq);
}

void grad_pull_bucket(const PeerPtrs& grads, const PeerPtrs& flags, int rank, int world, int bucket, int seq, int64_t lo,
                      int64_t n, float* out, bool accumulate, bool clear, bool handshake, int blocks, int* status,
                      cudaStream_t stream) {
  if (n == 0 || bucket < 0 || bucket >= kBucketSlots) return;
  if (blocks <= 0) blocks = 148 * 4;
  grad_pull_bucket_kernel<<<blocks, 512, 0, stream>>>(grads, flags, rank, world, bucket, seq, lo, n, out,
                                                      accumulate ? 1 : 0, clear ? 1 : 0, handshake ? 1 : 0, status);
}

void bucket_ready(const PeerPtrs& flags, int rank, int world, int bucket, int seq, int* status, cudaStream_t stream) {
  if (bucket < 0 || bucket >= kBucketSlots) return;
  bucket_ready_kernel<<<1, 32, 0, stream>>>(flags, rank, world, bucket, seq, status);
}

void adamw_publish(float* master, float* m, float* v, const float* grad, const PeerPtrs& params, int world, int64_t lo,
                   int64_t n, float lr, float b1, float b2, float eps, float wd, float bc1, float bc2,
                   float grad_scale, const float* clip_coef, cudaStream_t stream) {
  if (n == 0) return;
  adamw_publish_kernel<<<148 * 8, 256, 0, stream>>>(master, m, v, grad, params, world, lo, n, lr, b1, b2, eps, wd,
                                                    bc1, bc2, grad_scale, clip_coef);
}

}  // namespace mt
