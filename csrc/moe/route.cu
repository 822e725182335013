// MoE routing and dispatch kernels (sm_100a; bandwidth / latency bound, no tensor cores).
//
//  router_sigmoid_group   DeepSeek-V3 router: fp32 sigmoid scores, selection on score + bias, group score = sum of
//                         the two best experts of a group, keep `topk_group` groups, global top-k among them,
//                         weights = un-biased scores (optionally renormalised) * scaling.  One warp per token.
//  router_softmax_topk    fp32 softmax, top-k, optional renormalisation.  One warp per token.
//  router_*_bwd           gradient of the logits given d(weights) and d(scores).
//  moe_sort               stable counting sort of the N*K (token, slot) entries by expert: per-chunk histograms,
//                         a scan over chunks, and a one-warp-per-chunk ranking pass (match_any inside the warp, running
//                         counters in shared memory).  Produces group sizes, 128-row-padded offsets, the padded
//                         position of every entry and the inverse map padded row -> token.
//  moe_gather_rows        rows[p] = x[src[p] / K] * (w ? w[src[p]] : 1)  (zero rows where src < 0).
//  moe_combine_rows       out[n] = sum_k w[n,k] * y[pos[n,k]] ; optionally dw[n,k] = <y[pos[n,k]], g[n]>.
// Ties in top-k are broken towards the lower expert index, like a stable descending sort.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cstdint>
#include <stdexcept>
#include "../api.h"
#include "../common/bounds.cuh"

namespace mt {
namespace {

constexpr int kMaxPerLane = 16;  // experts per lane: E <= 512
constexpr int kMaxTopK = 16;
constexpr int kChunk = 2048;     // entries ranked by one warp

__device__ __forceinline__ void warp_argmax(float& v, int& i) {
#pragma unroll
  for (int m = 16; m > 0; m >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, m);
    const int oi = __shfl_xor_sync(0xffffffffu, i, m);
    if (ov > v || (ov == v && oi < i)) {
      v = ov;
      i = oi;
    }
  }
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int m = 16; m > 0; m >>= 1) v += __shfl_xor_sync(0xffffffffu, v, m);
  return v;
}

template <typename T>
__device__ __forceinline__ float to_f(T v);
template <>
__device__ __forceinline__ float to_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

// Lane l holds experts l, l+32, l+64, ...  `sel` is destroyed (chosen entries are set to -inf).
__device__ __forceinline__ void warp_topk(float (&sel)[kMaxPerLane], int per_lane, int E, int lane, int top_k,
                                          int (&out_idx)[kMaxTopK]) {
  for (int k = 0; k < top_k; ++k) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) {
      if (i < per_lane) {
        const int e = lane + 32 * i;
        if (e < E && (sel[i] > bv || (sel[i] == bv && e < bi))) {
          bv = sel[i];
          bi = e;
        }
      }
    }
    warp_argmax(bv, bi);
    out_idx[k] = bi;
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i)
      if (i < per_lane && lane + 32 * i == bi) sel[i] = -INFINITY;
  }
}

template <typename T>
__global__ void router_sigmoid_group_kernel(const T* __restrict__ logits, const float* __restrict__ bias,
                                            float* __restrict__ scores, int64_t* __restrict__ topk_idx,
                                            float* __restrict__ topk_w, int N, int E, int top_k, int n_group,
                                            int topk_group, int norm, float scaling) {
  extern __shared__ float sh[];  // per warp: E selection scores
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = blockIdx.x * (blockDim.x >> 5) + warp;
  if (n >= N) return;
  float* ssel = sh + warp * E;
  const int per_lane = (E + 31) / 32;
  float sc[kMaxPerLane], sel[kMaxPerLane];
#pragma unroll
  for (int i = 0; i < kMaxPerLane; ++i) {
    const int e = lane + 32 * i;
    sc[i] = 0.f;
    sel[i] = -INFINITY;
    if (i < per_lane && e < E) {
      const float s = 1.f / (1.f + __expf(-to_f(logits[(int64_t)n * E + e])));
      sc[i] = s;
      sel[i] = s + bias[e];
      scores[(int64_t)n * E + e] = s;
      ssel[e] = sel[i];
    }
  }
  __syncwarp();
  if (n_group > 1) {
    // group score (sum of the two best members), one group per lane (n_group <= 32)
    const int per = E / n_group;
    float gs = -INFINITY;
    if (lane < n_group) {
      float a = -INFINITY, b2 = -INFINITY;
      for (int j = 0; j < per; ++j) {
        const float v = ssel[lane * per + j];
        if (v > a) {
          b2 = a;
          a = v;
        } else if (v > b2) {
          b2 = v;
        }
      }
      gs = per >= 2 ? a + b2 : a;
    }
    // keep the topk_group best groups (lower index wins ties)
    unsigned keep = 0;
    for (int g = 0; g < topk_group; ++g) {
      float v = gs;
      int i = lane < n_group ? lane : 0x7fffffff;
      warp_argmax(v, i);
      keep |= 1u << i;
      if (lane == i) gs = -INFINITY;
    }
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) {
      const int e = lane + 32 * i;
      if (i < per_lane && e < E && !((keep >> (e / per)) & 1u)) sel[i] = -INFINITY;
    }
  }
  int idx[kMaxTopK];
  warp_topk(sel, per_lane, E, lane, top_k, idx);
  // weights: un-biased scores of the chosen experts (owner lane broadcasts)
  float wsum = 0.f;
  float w[kMaxTopK];
  for (int k = 0; k < top_k; ++k) {
    const int e = idx[k];
    float v = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i)
      if (i < per_lane && lane + 32 * i == e) v = sc[i];
    v = __shfl_sync(0xffffffffu, v, e & 31);
    w[k] = v;
    wsum += v;
  }
  const float inv = norm ? 1.f / (wsum + 1e-20f) : 1.f;
  if (lane == 0) {
    for (int k = 0; k < top_k; ++k) {
      topk_idx[(int64_t)n * top_k + k] = idx[k];
      topk_w[(int64_t)n * top_k + k] = w[k] * inv * scaling;
    }
  }
}

// dlogits[n,e] = (dscores[n,e] + ds_sel[n,e]) * s (1 - s), ds_sel from the chosen experts' weights.
__global__ void router_sigmoid_bwd_kernel(const float* __restrict__ scores, const int64_t* __restrict__ topk_idx,
                                          const float* __restrict__ dw, const float* __restrict__ dscores,
                                          float* __restrict__ dlogits, int N, int E, int top_k, int norm,
                                          float scaling) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = blockIdx.x * (blockDim.x >> 5) + warp;
  if (n >= N) return;
  const float* s = scores + (int64_t)n * E;
  float sk = 0.f, gk = 0.f;
  int ek = -1;
  if (lane < top_k) {
    ek = (int)topk_idx[(int64_t)n * top_k + lane];
    sk = s[ek];
    gk = dw ? dw[(int64_t)n * top_k + lane] * scaling : 0.f;
  }
  float ds = gk;
  if (norm) {
    const float sum = warp_sum(sk) + 1e-20f;
    const float dot = warp_sum(gk * sk);
    ds = gk / sum - dot / (sum * sum);
  }
  for (int e = lane; e < E; e += 32) {
    const float v = s[e];
    dlogits[(int64_t)n * E + e] = dscores ? dscores[(int64_t)n * E + e] * v * (1.f - v) : 0.f;
  }
  __syncwarp();
  if (lane < top_k) {
    const float v = sk;
    dlogits[(int64_t)n * E + ek] += ds * v * (1.f - v);  // chosen experts are distinct: no race
  }
}

template <typename T>
__global__ void router_softmax_topk_kernel(const T* __restrict__ logits, float* __restrict__ probs,
                                           int64_t* __restrict__ topk_idx, float* __restrict__ topk_w, int N, int E,
                                           int top_k, int norm, float scaling) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = blockIdx.x * (blockDim.x >> 5) + warp;
  if (n >= N) return;
  const int per_lane = (E + 31) / 32;
  float p[kMaxPerLane], sel[kMaxPerLane];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < kMaxPerLane; ++i) {
    const int e = lane + 32 * i;
    p[i] = -INFINITY;
    if (i < per_lane && e < E) p[i] = to_f(logits[(int64_t)n * E + e]);
    mx = fmaxf(mx, p[i]);
  }
#pragma unroll
  for (int m = 16; m > 0; m >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, m));
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < kMaxPerLane; ++i) {
    const int e = lane + 32 * i;
    p[i] = (i < per_lane && e < E) ? __expf(p[i] - mx) : 0.f;
    sum += p[i];
  }
  sum = warp_sum(sum);
  const float inv_sum = 1.f / sum;
#pragma unroll
  for (int i = 0; i < kMaxPerLane; ++i) {
    const int e = lane + 32 * i;
    p[i] *= inv_sum;
    sel[i] = (i < per_lane && e < E) ? p[i] : -INFINITY;
    if (i < per_lane && e < E) probs[(int64_t)n * E + e] = p[i];
  }
  int idx[kMaxTopK];
  warp_topk(sel, per_lane, E, lane, top_k, idx);
  float w[kMaxTopK];
  float wsum = 0.f;
  for (int k = 0; k < top_k; ++k) {
    const int e = idx[k];
    float v = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i)
      if (i < per_lane && lane + 32 * i == e) v = p[i];
    v = __shfl_sync(0xffffffffu, v, e & 31);
    w[k] = v;
    wsum += v;
  }
  const float inv = norm ? 1.f / (wsum + 1e-20f) : 1.f;
  if (lane == 0) {
    for (int k = 0; k < top_k; ++k) {
      topk_idx[(int64_t)n * top_k + k] = idx[k];
      topk_w[(int64_t)n * top_k + k] = w[k] * inv * scaling;
    }
  }
}

// g = dprobs + (gradient reaching the chosen probabilities through the weights); dlogits = p * (g - sum(g p)).
__global__ void router_softmax_bwd_kernel(const float* __restrict__ probs, const int64_t* __restrict__ topk_idx,
                                          const float* __restrict__ dw, const float* __restrict__ dprobs,
                                          float* __restrict__ dlogits, int N, int E, int top_k, int norm,
                                          float scaling) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = blockIdx.x * (blockDim.x >> 5) + warp;
  if (n >= N) return;
  const float* p = probs + (int64_t)n * E;
  float* g = dlogits + (int64_t)n * E;  // used as scratch for g first
  float pk = 0.f, gk = 0.f;
  int ek = -1;
  if (lane < top_k) {
    ek = (int)topk_idx[(int64_t)n * top_k + lane];
    pk = p[ek];
    gk = dw ? dw[(int64_t)n * top_k + lane] * scaling : 0.f;
  }
  float dp = gk;
  if (norm) {
    const float sum = warp_sum(pk) + 1e-20f;
    const float dot = warp_sum(gk * pk);
    dp = gk / sum - dot / (sum * sum);
  }
  for (int e = lane; e < E; e += 32) g[e] = dprobs ? dprobs[(int64_t)n * E + e] : 0.f;
  __syncwarp();
  if (lane < top_k) g[ek] += dp;
  __syncwarp();
  float dot = 0.f;
  for (int e = lane; e < E; e += 32) dot += g[e] * p[e];
  dot = warp_sum(dot);
  for (int e = lane; e < E; e += 32) g[e] = p[e] * (g[e] - dot);
}

// ------------------------------------------------------------------------------------------ counting sort
__global__ void moe_count_kernel(const int64_t* __restrict__ experts, int M, int E, int* __restrict__ chunk_counts) {
  extern __shared__ int cnt[];
  for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  const int base = blockIdx.x * kChunk;
  for (int i = threadIdx.x; i < kChunk && base + i < M; i += blockDim.x)
    if (MT_IN_BOUNDS(experts[base + i], E)) atomicAdd(&cnt[(int)experts[base + i]], 1);
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) chunk_counts[blockIdx.x * E + e] = cnt[e];
}

// One block: per expert, exclusive scan over chunks (chunk_counts becomes the chunk's start inside the expert's group),
// group sizes, then 128-padded offsets.
__global__ void moe_scan_kernel(int* __restrict__ chunk_counts, int nchunks, int E, int64_t* __restrict__ sizes,
                                int* __restrict__ off_p) {
  extern __shared__ int tot[];
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int run = 0;
    for (int c = 0; c < nchunks; ++c) {
      const int v = chunk_counts[c * E + e];
      chunk_counts[c * E + e] = run;
      run += v;
    }
    tot[e] = run;
    sizes[e] = run;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int e = 0; e < E; ++e) {
      off_p[e] = run;
      run += (tot[e] + 127) / 128 * 128;
    }
    off_p[E] = run;
  }
}

// One warp per chunk walks its entries in order, 32 at a time: the rank of an entry inside its expert's group is the
// running count of that expert (chunk start + entries seen so far) plus the number of lower lanes with the same expert.
__global__ void moe_rank_kernel(const int64_t* __restrict__ experts, int M, int E,
                                const int* __restrict__ chunk_starts, const int* __restrict__ off_p,
                                int64_t* __restrict__ pos, int* __restrict__ src) {
  extern __shared__ int run[];
  const int lane = threadIdx.x;
  for (int e = lane; e < E; e += 32) run[e] = off_p[e] + chunk_starts[blockIdx.x * E + e];
  __syncwarp();
  const int base = blockIdx.x * kChunk;
  for (int i0 = 0; i0 < kChunk && base + i0 < M; i0 += 32) {
    const int i = base + i0 + lane;
    const bool live = i < M && MT_IN_BOUNDS(experts[i < M ? i : 0], E);
    const int e = live ? (int)experts[i] : -1 - lane;  // dead lanes match nobody
    const unsigned peers = __match_any_sync(0xffffffffu, e);
    const int before = __popc(peers & ((1u << lane) - 1u));
    int start = 0;
    if (live) start = run[e];
    __syncwarp();
    if (live) {
      const int p = start + before;
      pos[i] = p;
      src[p] = i;
      if (before == __popc(peers) - 1) run[e] = start + before + 1;  // last peer advances the counter
    }
    __syncwarp();
  }
}

union Pack8 {
  uint4 u;
  __nv_bfloat16 h[8];
};

// rows[p, :] = scale * x[src[p] / K, :] (zeros where src[p] < 0; src holds flat (token, slot) entries);
// scale = w[src[p]] when w is given.
__global__ void moe_gather_rows_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ src,
                                       const float* __restrict__ w, __nv_bfloat16* __restrict__ rows, int64_t cap,
                                       int K, int D, int64_t entries) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int vecs = D >> 3;
  for (int64_t p = (int64_t)blockIdx.x * (blockDim.x >> 5) + warp; p < cap; p += (int64_t)gridDim.x * (blockDim.x >> 5)) {
    const int s = src[p];
    uint4* dst = reinterpret_cast<uint4*>(rows + p * D);
    if (s < 0 || !MT_IN_BOUNDS(s, entries)) {
      for (int v = lane; v < vecs; v += 32) dst[v] = make_uint4(0, 0, 0, 0);
      continue;
    }
    const uint4* in = reinterpret_cast<const uint4*>(x + (int64_t)(s / K) * D);
    if (w == nullptr) {
      for (int v = lane; v < vecs; v += 32) dst[v] = in[v];
    } else {
      const float sc = w[s];
      for (int v = lane; v < vecs; v += 32) {
        Pack8 a;
        a.u = in[v];
#pragma unroll
        for (int j = 0; j < 8; ++j) a.h[j] = __float2bfloat16(__bfloat162float(a.h[j]) * sc);
        dst[v] = a.u;
      }
    }
  }
}

// out[n, :] = sum_k w[n,k] * y[pos[n,k], :]  (w == nullptr: plain sum); dw[n,k] = <y[pos[n,k], :], g[n, :]> if asked.
// A negative position marks a dropped (token, slot): its row is never read, it adds nothing and its dw is 0.
template <int KMAX>
__global__ void moe_combine_rows_kernel(const __nv_bfloat16* __restrict__ y, const int64_t* __restrict__ pos,
                                        const float* __restrict__ w, __nv_bfloat16* __restrict__ out,
                                        const __nv_bfloat16* __restrict__ g, float* __restrict__ dw, int N, int K,
                                        int D, int64_t y_rows) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int vecs = D >> 3;
  for (int n = blockIdx.x * (blockDim.x >> 5) + warp; n < N; n += gridDim.x * (blockDim.x >> 5)) {
    int64_t pk[KMAX];
    float wk[KMAX];
#pragma unroll
    for (int k = 0; k < KMAX; ++k) {
      pk[k] = k < K ? pos[(int64_t)n * K + k] : 0;
      if (pk[k] >= 0 && !MT_IN_BOUNDS(pk[k], y_rows)) pk[k] = -1;  // reported; treated like a dropped slot
      wk[k] = k < K ? (w ? w[(int64_t)n * K + k] : 1.f) : 0.f;
    }
    if (out != nullptr) {
      for (int v = lane; v < vecs; v += 32) {
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
        for (int k = 0; k < KMAX; ++k) {
          if (k < K && pk[k] >= 0) {
            Pack8 a;
            a.u = reinterpret_cast<const uint4*>(y + pk[k] * D)[v];
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] += wk[k] * __bfloat162float(a.h[j]);
          }
        }
        Pack8 o;
#pragma unroll
        for (int j = 0; j < 8; ++j) o.h[j] = __float2bfloat16(acc[j]);
        reinterpret_cast<uint4*>(out + (int64_t)n * D)[v] = o.u;
      }
    }
    if (dw != nullptr) {
#pragma unroll
      for (int k = 0; k < KMAX; ++k) {
        if (k < K) {
          float dot = 0.f;
          for (int v = lane; v < vecs && pk[k] >= 0; v += 32) {
            Pack8 a, b;
            a.u = reinterpret_cast<const uint4*>(y + pk[k] * D)[v];
            b.u = reinterpret_cast<const uint4*>(g + (int64_t)n * D)[v];
#pragma unroll
            for (int j = 0; j < 8; ++j) dot += __bfloat162float(a.h[j]) * __bfloat162float(b.h[j]);
          }
          dot = warp_sum(dot);
          if (lane == 0) dw[(int64_t)n * K + k] = dot;
        }
      }
    }
  }
}

void check_router_args(int E, int top_k, int n_group) {
  if (E > 32 * kMaxPerLane) throw std::runtime_error("router: at most 512 experts");
  if (top_k > kMaxTopK || top_k > 32) throw std::runtime_error("router: top_k must be <= 16");
  if (n_group > 32 || (n_group > 0 && E % n_group != 0)) throw std::runtime_error("router: bad n_group");
}

}  // namespace

void router_sigmoid_group(const void* logits, bool logits_bf16, const float* bias, float* scores, int64_t* topk_idx,
                          float* topk_w, int N, int E, int top_k, int n_group, int topk_group, bool norm, float scaling,
                          cudaStream_t stream) {
  check_router_args(E, top_k, n_group);
  if (N == 0) return;
  const int warps = 4;
  const int grid = (N + warps - 1) / warps;
  const size_t sh = (size_t)warps * E * sizeof(float);
  if (logits_bf16)
    router_sigmoid_group_kernel<__nv_bfloat16><<<grid, warps * 32, sh, stream>>>(
        (const __nv_bfloat16*)logits, bias, scores, topk_idx, topk_w, N, E, top_k, n_group, topk_group, norm, scaling);
  else
    router_sigmoid_group_kernel<float><<<grid, warps * 32, sh, stream>>>(
        (const float*)logits, bias, scores, topk_idx, topk_w, N, E, top_k, n_group, topk_group, norm, scaling);
}

void router_softmax_topk(const void* logits, bool logits_bf16, float* probs, int64_t* topk_idx, float* topk_w, int N,
                         int E, int top_k, bool norm, float scaling, cudaStream_t stream) {
  check_router_args(E, top_k, 0);
  if (N == 0) return;
  const int warps = 4;
  const int grid = (N + warps - 1) / warps;
  if (logits_bf16)
    router_softmax_topk_kernel<__nv_bfloat16><<<grid, warps * 32, 0, stream>>>((const __nv_bfloat16*)logits, probs,
                                                                               topk_idx, topk_w, N, E, top_k, norm, scaling);
  else
    router_softmax_topk_kernel<float><<<grid, warps * 32, 0, stream>>>((const float*)logits, probs, topk_idx, topk_w, N,
                                                                       E, top_k, norm, scaling);
}

void router_bwd(bool softmax, const float* scores, const int64_t* topk_idx, const float* dw, const float* dscores,
                float* dlogits, int N, int E, int top_k, bool norm, float scaling, cudaStream_t stream) {
  if (N == 0) return;
  const int warps = 4;
  const int grid = (N + warps - 1) / warps;
  if (softmax)
    router_softmax_bwd_kernel<<<grid, warps * 32, 0, stream>>>(scores, topk_idx, dw, dscores, dlogits, N, E, top_k, norm,
                                                               scaling);
  else
    router_sigmoid_bwd_kernel<<<grid, warps * 32, 0, stream>>>(scores, topk_idx, dw, dscores, dlogits, N, E, top_k, norm,
                                                               scaling);
}

int moe_sort_chunks(int M) { return (M + kChunk - 1) / kChunk; }

void moe_sort(const int64_t* experts, int M, int E, int64_t cap, int* chunk_counts, int64_t* sizes, int* off_p,
              int64_t* pos, int* src, cudaStream_t stream) {
  const int nchunks = moe_sort_chunks(M);
  cudaMemsetAsync(src, 0xff, (size_t)cap * sizeof(int), stream);  // -1: padding row
  if (nchunks > 0) moe_count_kernel<<<nchunks, 256, E * sizeof(int), stream>>>(experts, M, E, chunk_counts);
  moe_scan_kernel<<<1, 256, E * sizeof(int), stream>>>(chunk_counts, nchunks, E, sizes, off_p);
  if (nchunks > 0) moe_rank_kernel<<<nchunks, 32, E * sizeof(int), stream>>>(experts, M, E, chunk_counts, off_p, pos, src);
}

void moe_gather_rows(const void* x, const int* src, const float* w, void* rows, int64_t cap, int K, int D,
                     int64_t entries, cudaStream_t stream) {
  if (cap == 0) return;
  int64_t blocks = (cap + 7) / 8;
  if (blocks > 148 * 32) blocks = 148 * 32;
  moe_gather_rows_kernel<<<(int)blocks, 256, 0, stream>>>((const __nv_bfloat16*)x, src, w, (__nv_bfloat16*)rows, cap, K, D,
                                                          entries);
}

void moe_combine_rows(const void* y, const int64_t* pos, const float* w, void* out, const void* g, float* dw, int N,
                      int K, int D, int64_t y_rows, cudaStream_t stream) {
  if (N == 0) return;
  if (K > 16) throw std::runtime_error("moe_combine_rows: top_k must be <= 16");
  int blocks = (N + 7) / 8;
  if (blocks > 148 * 32) blocks = 148 * 32;
  auto y_ = (const __nv_bfloat16*)y;
  auto o_ = (__nv_bfloat16*)out;
  auto g_ = (const __nv_bfloat16*)g;
  if (K <= 2) moe_combine_rows_kernel<2><<<blocks, 256, 0, stream>>>(y_, pos, w, o_, g_, dw, N, K, D, y_rows);
  else if (K <= 4) moe_combine_rows_kernel<4><<<blocks, 256, 0, stream>>>(y_, pos, w, o_, g_, dw, N, K, D, y_rows);
  else if (K <= 8) moe_combine_rows_kernel<8><<<blocks, 256, 0, stream>>>(y_, pos, w, o_, g_, dw, N, K, D, y_rows);
  else moe_combine_rows_kernel<16><<<blocks, 256, 0, stream>>>(y_, pos, w, o_, g_, dw, N, K, D, y_rows);
}

}  // namespace mt
