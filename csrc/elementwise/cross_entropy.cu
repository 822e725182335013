// Softmax cross-entropy over bf16 logits with label smoothing, z-loss and optional tanh soft-capping.
// One CTA per row: pass 1 keeps an online (max, sum-exp, sum-logit) triple, pass 2 overwrites the row with
//   dlogits = grad_scale * [ softmax * (1 + 2 w lse) - ls/V - (1 - ls) * onehot ]  (times the soft-cap slope)
// so the [rows, V] fp32 logits / probabilities are never materialised.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cfloat>
#include <cstdint>
#include "../api.h"
#include "../common/bounds.cuh"

namespace mt {
namespace {

constexpr int kThreads = 512;

union Pack8 {
  uint4 u;
  __nv_bfloat16 h[8];
};

struct Triple {
  float m, s, t;  // running max, sum exp(x - m), sum x
};

__device__ __forceinline__ Triple combine(Triple a, Triple b) {
  Triple r;
  r.m = fmaxf(a.m, b.m);
  r.s = (a.m == -FLT_MAX ? 0.f : a.s * __expf(a.m - r.m)) + (b.m == -FLT_MAX ? 0.f : b.s * __expf(b.m - r.m));
  r.t = a.t + b.t;
  return r;
}

__device__ __forceinline__ float cap(float x, float softcap) { return softcap > 0.f ? tanhf(x / softcap) * softcap : x; }

__global__ void __launch_bounds__(kThreads)
ce_kernel(__nv_bfloat16* __restrict__ logits, const int64_t* __restrict__ targets, float* __restrict__ loss,
          float* __restrict__ zloss, float* __restrict__ lse_out, int V, int64_t ldl, float ls, float zw,
          float softcap, float grad_scale, int write_grad) {
  __shared__ Triple red[kThreads / 32];
  __shared__ Triple total;
  const int64_t row = blockIdx.x;
  __nv_bfloat16* lr = logits + row * ldl;
  const int nvec = V >> 3;
  Triple acc = {-FLT_MAX, 0.f, 0.f};
  for (int i = threadIdx.x; i < nvec; i += kThreads) {
    Pack8 a;
    a.u = reinterpret_cast<const uint4*>(lr)[i];
    // one rescale of the running sum per vector (9 exponentials for 8 elements instead of 16): the kernel is
    // bound by the exponential unit, not by memory
    float x[8];
    float vm = -FLT_MAX;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      x[j] = cap(__bfloat162float(a.h[j]), softcap);
      vm = fmaxf(vm, x[j]);
    }
    const float nm = fmaxf(acc.m, vm);
    float vs = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      vs += __expf(x[j] - nm);
      acc.t += x[j];
    }
    acc.s = acc.s * __expf(acc.m - nm) + vs;
    acc.m = nm;
  }
  for (int i = (nvec << 3) + threadIdx.x; i < V; i += kThreads) {
    const float x = cap(__bfloat162float(lr[i]), softcap);
    const float nm = fmaxf(acc.m, x);
    acc.s = acc.s * __expf(acc.m - nm) + __expf(x - nm);
    acc.m = nm;
    acc.t += x;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    Triple b;
    b.m = __shfl_xor_sync(0xffffffffu, acc.m, o);
    b.s = __shfl_xor_sync(0xffffffffu, acc.s, o);
    b.t = __shfl_xor_sync(0xffffffffu, acc.t, o);
    acc = combine(acc, b);
  }
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    Triple r = red[0];
    for (int w = 1; w < kThreads / 32; ++w) r = combine(r, red[w]);
    total = r;
  }
  __syncthreads();
  const float lse = total.m + logf(total.s);
  int64_t tgt = targets[row];
  if (!MT_IN_BOUNDS(tgt, V)) tgt = 0;  // debug-bounds build: reported; the row then scores class 0 instead of faulting
  if (threadIdx.x == 0) {
    const float xt = cap(__bfloat162float(lr[tgt]), softcap);
    const float nll = lse - xt;
    const float smooth = lse - total.t / V;
    loss[row] = (1.f - ls) * nll + ls * smooth + zw * lse * lse;
    if (zloss) zloss[row] = zw * lse * lse;
    if (lse_out) lse_out[row] = lse;
  }
  if (!write_grad) return;
  __syncthreads();  // the target logit was read above before anyone overwrites the row
  const float zfac = 1.f + 2.f * zw * lse;
  const float lsv = ls / V;
  for (int i = threadIdx.x; i < nvec; i += kThreads) {
    Pack8 a;
    a.u = reinterpret_cast<const uint4*>(lr)[i];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float raw = __bfloat162float(a.h[j]);
      const float x = cap(raw, softcap);
      float g = __expf(x - lse) * zfac - lsv;
      if ((int64_t)(i * 8 + j) == tgt) g -= (1.f - ls);
      if (softcap > 0.f) {
        const float th = x / softcap;
        g *= (1.f - th * th);
      }
      a.h[j] = __float2bfloat16(g * grad_scale);
    }
    reinterpret_cast<uint4*>(lr)[i] = a.u;
  }
  for (int i = (nvec << 3) + threadIdx.x; i < V; i += kThreads) {
    const float raw = __bfloat162float(lr[i]);
    const float x = cap(raw, softcap);
    float g = __expf(x - lse) * zfac - lsv;
    if ((int64_t)i == tgt) g -= (1.f - ls);
    if (softcap > 0.f) {
      const float th = x / softcap;
      g *= (1.f - th * th);
    }
    lr[i] = __float2bfloat16(g * grad_scale);
  }
}

}  // namespace

void cross_entropy_fwd_bwd(void* logits, const int64_t* targets, float* loss, float* zloss, float* lse,
                           int64_t rows, int V, int64_t ldl, float label_smoothing, float z_weight, float softcap,
                           float grad_scale, bool write_grad, cudaStream_t stream) {
  if (rows == 0) return;
  ce_kernel<<<(unsigned)rows, kThreads, 0, stream>>>((__nv_bfloat16*)logits, targets, loss, zloss, lse, V, ldl,
                                                     label_smoothing, z_weight, softcap, grad_scale,
                                                     write_grad ? 1 : 0);
}

}  // namespace mt
