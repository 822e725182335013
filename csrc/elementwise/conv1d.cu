// Depth-wise causal conv1d fused with SiLU, forward and backward (bf16 in/out, fp32 math), for the short
// convolution of the Gated Delta Rule layers:
//     pre[b,s,c] = sum_j w[c,j] * x[b, s-(K-1)+j, c]      y = silu(pre)
// A thread owns 8 adjacent channels (one 16-byte vector) and walks a run of consecutive tokens with the last K-1
// inputs in registers, so every input is read once (plus the K-1 token halo per run).  Backward recomputes `pre`,
// forms dpre = dy * silu'(pre), the anti-causal data gradient and per-thread weight-gradient partials that are
// reduced over the block's runs in shared memory before one atomic add per (channel, tap).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cstdint>
#include <stdexcept>
#include "../api.h"

namespace mt {
namespace {

constexpr int kRun = 16;       // tokens per thread run
constexpr int kWarps = 8;      // runs per block

union Pack8 {
  uint4 u;
  __nv_bfloat16 h[8];
};

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&v)[8]) {
  Pack8 a;
  a.u = *reinterpret_cast<const uint4*>(p);
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = __bfloat162float(a.h[i]);
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&v)[8]) {
  Pack8 a;
#pragma unroll
  for (int i = 0; i < 8; ++i) a.h[i] = __float2bfloat16(v[i]);
  *reinterpret_cast<uint4*>(p) = a.u;
}
__device__ __forceinline__ float silu(float x) { return x / (1.f + __expf(-x)); }
__device__ __forceinline__ float dsilu(float x) {
  const float s = 1.f / (1.f + __expf(-x));
  return s * (1.f + x * (1.f - s));
}

template <int K>
__global__ void conv1d_silu_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                       __nv_bfloat16* __restrict__ y, int B, int S, int C) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int c0 = (blockIdx.x * 32 + lane) * 8;
  const int runs_per_seq = (S + kRun - 1) / kRun;
  const int run = blockIdx.y * kWarps + warp;
  if (c0 >= C || run >= B * runs_per_seq) return;
  const int b = run / runs_per_seq;
  const int s0 = (run % runs_per_seq) * kRun;
  float wt[K][8];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < K; ++j) wt[j][i] = __bfloat162float(w[(c0 + i) * K + j]);
  const __nv_bfloat16* xb = x + (int64_t)b * S * C + c0;
  __nv_bfloat16* yb = y + (int64_t)b * S * C + c0;
  float win[K][8];  // win[j] = x(s - (K-1) + j)
#pragma unroll
  for (int j = 0; j < K - 1; ++j) {
    const int s = s0 - (K - 1) + j;
    if (s >= 0) load8(xb + (int64_t)s * C, win[j + 1]);
    else
#pragma unroll
      for (int i = 0; i < 8; ++i) win[j + 1][i] = 0.f;
  }
  const int s_end = min(s0 + kRun, S);
#pragma unroll 4
  for (int s = s0; s < s_end; ++s) {
#pragma unroll
    for (int j = 0; j < K - 1; ++j)
#pragma unroll
      for (int i = 0; i < 8; ++i) win[j][i] = win[j + 1][i];
    load8(xb + (int64_t)s * C, win[K - 1]);
    float out[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float acc = 0.f;
#pragma unroll
      for (int j = 0; j < K; ++j) acc = fmaf(wt[j][i], win[j][i], acc);
      out[i] = silu(acc);
    }
    store8(yb + (int64_t)s * C, out);
  }
}

template <int K>
__global__ void conv1d_silu_bwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                       const __nv_bfloat16* __restrict__ dy, __nv_bfloat16* __restrict__ dx,
                                       float* __restrict__ dw, int B, int S, int C) {
  __shared__ float red[kWarps][32][8];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int c0 = (blockIdx.x * 32 + lane) * 8;
  const int runs_per_seq = (S + kRun - 1) / kRun;
  const int run = blockIdx.y * kWarps + warp;
  const bool live = c0 < C && run < B * runs_per_seq;
  float dwt[K][8];
#pragma unroll
  for (int j = 0; j < K; ++j)
#pragma unroll
    for (int i = 0; i < 8; ++i) dwt[j][i] = 0.f;
  if (live) {
    const int b = run / runs_per_seq;
    const int s0 = (run % runs_per_seq) * kRun;
    float wt[K][8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int j = 0; j < K; ++j) wt[j][i] = __bfloat162float(w[(c0 + i) * K + j]);
    const __nv_bfloat16* xb = x + (int64_t)b * S * C + c0;
    const __nv_bfloat16* gb = dy + (int64_t)b * S * C + c0;
    __nv_bfloat16* dxb = dx + (int64_t)b * S * C + c0;
    float win[K][8];   // inputs x(s-(K-1)) .. x(s)
    float ring[K][8];  // ring[j] = dpre(s - j)
#pragma unroll
    for (int j = 0; j < K; ++j)
#pragma unroll
      for (int i = 0; i < 8; ++i) ring[j][i] = 0.f;
#pragma unroll
    for (int j = 0; j < K - 1; ++j) {
      const int s = s0 - (K - 1) + j;
      if (s >= 0) load8(xb + (int64_t)s * C, win[j + 1]);
      else
#pragma unroll
        for (int i = 0; i < 8; ++i) win[j + 1][i] = 0.f;
    }
    const int s_run_end = min(s0 + kRun, S);
    const int s_last = s_run_end + (K - 1);  // dpre is needed K-1 tokens past the run for the run's last dx
#pragma unroll 2
    for (int s = s0; s < s_last; ++s) {
#pragma unroll
      for (int j = K - 1; j > 0; --j)
#pragma unroll
        for (int i = 0; i < 8; ++i) ring[j][i] = ring[j - 1][i];
#pragma unroll
      for (int j = 0; j < K - 1; ++j)
#pragma unroll
        for (int i = 0; i < 8; ++i) win[j][i] = win[j + 1][i];
      if (s < S) {
        load8(xb + (int64_t)s * C, win[K - 1]);
        float g[8];
        load8(gb + (int64_t)s * C, g);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          float acc = 0.f;
#pragma unroll
          for (int j = 0; j < K; ++j) acc = fmaf(wt[j][i], win[j][i], acc);
          ring[0][i] = g[i] * dsilu(acc);
        }
        if (s < s_run_end) {
#pragma unroll
          for (int j = 0; j < K; ++j)
#pragma unroll
            for (int i = 0; i < 8; ++i) dwt[j][i] = fmaf(ring[0][i], win[j][i], dwt[j][i]);
        }
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          ring[0][i] = 0.f;
          win[K - 1][i] = 0.f;
        }
      }
      const int t = s - (K - 1);  // dx(t) = sum_j w[j] * dpre(t + K-1-j) = sum_j w[j] * ring[j]
      if (t >= s0 && t < s_run_end) {
        float out[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          float acc = 0.f;
#pragma unroll
          for (int j = 0; j < K; ++j) acc = fmaf(wt[j][i], ring[j][i], acc);
          out[i] = acc;
        }
        store8(dxb + (int64_t)t * C, out);
      }
    }
  }
  // reduce the weight-gradient partials over the block's runs, one tap at a time
#pragma unroll
  for (int j = 0; j < K; ++j) {
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 8; ++i) red[warp][lane][i] = dwt[j][i];
    __syncthreads();
    if (warp == 0 && c0 < C) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float acc = 0.f;
#pragma unroll
        for (int r = 0; r < kWarps; ++r) acc += red[r][lane][i];
        atomicAdd(&dw[(c0 + i) * K + j], acc);
      }
    }
  }
}

template <int K>
void launch(const void* x, const void* w, const void* dy, void* out, float* dw, int B, int S, int C, bool bwd,
            cudaStream_t stream) {
  const int runs = B * ((S + kRun - 1) / kRun);
  dim3 grid((C / 8 + 31) / 32, (runs + kWarps - 1) / kWarps);
  if (!bwd)
    conv1d_silu_fwd_kernel<K><<<grid, kWarps * 32, 0, stream>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)w,
                                                                (__nv_bfloat16*)out, B, S, C);
  else
    conv1d_silu_bwd_kernel<K><<<grid, kWarps * 32, 0, stream>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)w,
                                                                (const __nv_bfloat16*)dy, (__nv_bfloat16*)out, dw, B, S, C);
}

void dispatch(int K, const void* x, const void* w, const void* dy, void* out, float* dw, int B, int S, int C, bool bwd,
              cudaStream_t stream) {
  if (C % 8 != 0) throw std::runtime_error("conv1d_silu: channels must be a multiple of 8");
  if (B * S == 0) return;
  switch (K) {
    case 2: launch<2>(x, w, dy, out, dw, B, S, C, bwd, stream); break;
    case 3: launch<3>(x, w, dy, out, dw, B, S, C, bwd, stream); break;
    case 4: launch<4>(x, w, dy, out, dw, B, S, C, bwd, stream); break;
    default: throw std::runtime_error("conv1d_silu: kernel width must be 2, 3 or 4");
  }
}

}  // namespace

void conv1d_silu_fwd(const void* x, const void* w, void* y, int B, int S, int C, int K, cudaStream_t stream) {
  dispatch(K, x, w, nullptr, y, nullptr, B, S, C, false, stream);
}

// dw (fp32 [C, K]) is accumulated into: zero it first unless accumulation is wanted.
void conv1d_silu_bwd(const void* x, const void* w, const void* dy, void* dx, float* dw, int B, int S, int C, int K,
                     cudaStream_t stream) {
  dispatch(K, x, w, dy, dx, dw, B, S, C, true, stream);
}

}  // namespace mt
