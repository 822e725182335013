// Gated activation  out = act(gate) * up  on the two column halves of a fused [rows, 2*inter] projection,
// and its backward.  bf16 I/O, fp32 math, 16-byte vectors.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cstdint>
#include "../api.h"

namespace mt {
namespace {

union Pack8 {
  uint4 u;
  __nv_bfloat16 h[8];
};

template <int ACT>
__device__ __forceinline__ void act_and_grad(float x, float& f, float& df) {
  if (ACT == 0) {  // silu
    const float s = 1.f / (1.f + __expf(-x));
    f = x * s;
    df = s * (1.f + x * (1.f - s));
  } else if (ACT == 1) {  // gelu, tanh approximation
    const float k0 = 0.7978845608028654f, k1 = 0.044715f;
    const float u = k0 * (x + k1 * x * x * x);
    const float t = tanhf(u);
    f = 0.5f * x * (1.f + t);
    df = 0.5f * (1.f + t) + 0.5f * x * (1.f - t * t) * k0 * (1.f + 3.f * k1 * x * x);
  } else if (ACT == 2) {  // gelu, exact
    const float c = 0.7071067811865476f;
    const float e = erff(x * c);
    f = 0.5f * x * (1.f + e);
    df = 0.5f * (1.f + e) + x * 0.3989422804014327f * __expf(-0.5f * x * x);
  } else {  // relu
    f = x > 0.f ? x : 0.f;
    df = x > 0.f ? 1.f : 0.f;
  }
}

template <int ACT>
__global__ void gated_fwd_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out, int64_t rows,
                                 int inter) {
  const int nvec = inter >> 3;
  const int64_t total = rows * nvec;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = idx / nvec;
    const int c = (int)(idx % nvec);
    Pack8 g, u, o;
    g.u = reinterpret_cast<const uint4*>(gu + r * 2 * inter)[c];
    u.u = reinterpret_cast<const uint4*>(gu + r * 2 * inter + inter)[c];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float f, df;
      act_and_grad<ACT>(__bfloat162float(g.h[j]), f, df);
      o.h[j] = __float2bfloat16(f * __bfloat162float(u.h[j]));
    }
    reinterpret_cast<uint4*>(out + r * inter)[c] = o.u;
  }
}

template <int ACT>
__global__ void gated_bwd_kernel(const __nv_bfloat16* __restrict__ gu, const __nv_bfloat16* __restrict__ dout,
                                 __nv_bfloat16* __restrict__ dgu, int64_t rows, int inter) {
  const int nvec = inter >> 3;
  const int64_t total = rows * nvec;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = idx / nvec;
    const int c = (int)(idx % nvec);
    Pack8 g, u, d, dg, du;
    g.u = reinterpret_cast<const uint4*>(gu + r * 2 * inter)[c];
    u.u = reinterpret_cast<const uint4*>(gu + r * 2 * inter + inter)[c];
    d.u = reinterpret_cast<const uint4*>(dout + r * inter)[c];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float f, df;
      act_and_grad<ACT>(__bfloat162float(g.h[j]), f, df);
      const float dd = __bfloat162float(d.h[j]);
      dg.h[j] = __float2bfloat16(dd * __bfloat162float(u.h[j]) * df);
      du.h[j] = __float2bfloat16(dd * f);
    }
    reinterpret_cast<uint4*>(dgu + r * 2 * inter)[c] = dg.u;
    reinterpret_cast<uint4*>(dgu + r * 2 * inter + inter)[c] = du.u;
  }
}

inline int grid_for(int64_t total) {
  int64_t b = (total + 255) / 256;
  return (int)(b > 148 * 32 ? 148 * 32 : b);
}

}  // namespace

void gated_act_fwd(const void* gate_up, void* out, int64_t rows, int inter, int act, cudaStream_t stream) {
  const int64_t total = rows * (inter / 8);
  if (total == 0) return;
  auto a = (const __nv_bfloat16*)gate_up;
  auto o = (__nv_bfloat16*)out;
  const int g = grid_for(total);
  switch (act) {
    case 0: gated_fwd_kernel<0><<<g, 256, 0, stream>>>(a, o, rows, inter); break;
    case 1: gated_fwd_kernel<1><<<g, 256, 0, stream>>>(a, o, rows, inter); break;
    case 2: gated_fwd_kernel<2><<<g, 256, 0, stream>>>(a, o, rows, inter); break;
    default: gated_fwd_kernel<3><<<g, 256, 0, stream>>>(a, o, rows, inter); break;
  }
}

void gated_act_bwd(const void* gate_up, const void* dout, void* dgate_up, int64_t rows, int inter, int act,
                   cudaStream_t stream) {
  const int64_t total = rows * (inter / 8);
  if (total == 0) return;
  auto a = (const __nv_bfloat16*)gate_up;
  auto d = (const __nv_bfloat16*)dout;
  auto o = (__nv_bfloat16*)dgate_up;
  const int g = grid_for(total);
  switch (act) {
    case 0: gated_bwd_kernel<0><<<g, 256, 0, stream>>>(a, d, o, rows, inter); break;
    case 1: gated_bwd_kernel<1><<<g, 256, 0, stream>>>(a, d, o, rows, inter); break;
    case 2: gated_bwd_kernel<2><<<g, 256, 0, stream>>>(a, d, o, rows, inter); break;
    default: gated_bwd_kernel<3><<<g, 256, 0, stream>>>(a, d, o, rows, inter); break;
  }
}

}  // namespace mt
