// Gated activation  out = act(gate) * up  on the two column halves of a fused [rows, 2*inter] projection,
// and its backward.  bf16 I/O, fp32 math, 16-byte vectors.
// Also  out = x * f(gate)  with x and gate in separate, row-strided tensors: f = sigmoid is the attention output gate
// (mintext/modules/attention.py:361-362), f = silu the gate after the per-head norm of the Gated Delta Rule layers
// (mintext/modules/linear_attention.py:375-376); the strides let the gate be a column block of a fused projection.
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

// MODE 0: f = sigmoid, MODE 1: f = silu
template <int MODE>
__device__ __forceinline__ void gate_fn(float g, float& f, float& df) {
  const float s = 1.f / (1.f + __expf(-g));
  if (MODE == 0) {
    f = s;
    df = s * (1.f - s);
  } else {
    f = g * s;
    df = s * (1.f + g * (1.f - s));
  }
}

template <int MODE>
__global__ void gate_mul_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ gate,
                                    __nv_bfloat16* __restrict__ out, int64_t rows, int dim, int64_t xs, int64_t gs) {
  const int nvec = dim >> 3;
  const int64_t total = rows * nvec;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = idx / nvec;
    const int c = (int)(idx % nvec);
    Pack8 a, g, o;
    a.u = reinterpret_cast<const uint4*>(x + r * xs)[c];
    g.u = reinterpret_cast<const uint4*>(gate + r * gs)[c];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float f, df;
      gate_fn<MODE>(__bfloat162float(g.h[j]), f, df);
      o.h[j] = __float2bfloat16(__bfloat162float(a.h[j]) * f);
    }
    reinterpret_cast<uint4*>(out + r * dim)[c] = o.u;
  }
}

template <int MODE>
__global__ void gate_mul_bwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ gate,
                                    const __nv_bfloat16* __restrict__ dout, __nv_bfloat16* __restrict__ dx,
                                    __nv_bfloat16* __restrict__ dgate, int64_t rows, int dim, int64_t xs, int64_t gs) {
  const int nvec = dim >> 3;
  const int64_t total = rows * nvec;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = idx / nvec;
    const int c = (int)(idx % nvec);
    Pack8 a, g, d, da, dg;
    a.u = reinterpret_cast<const uint4*>(x + r * xs)[c];
    g.u = reinterpret_cast<const uint4*>(gate + r * gs)[c];
    d.u = reinterpret_cast<const uint4*>(dout + r * dim)[c];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float f, df;
      gate_fn<MODE>(__bfloat162float(g.h[j]), f, df);
      const float dd = __bfloat162float(d.h[j]);
      da.h[j] = __float2bfloat16(dd * f);
      dg.h[j] = __float2bfloat16(dd * __bfloat162float(a.h[j]) * df);
    }
    reinterpret_cast<uint4*>(dx + r * dim)[c] = da.u;
    reinterpret_cast<uint4*>(dgate + r * dim)[c] = dg.u;
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

// x, gate: rows of `dim` bf16 at row pitches xs, gs (elements); out, dx, dgate: contiguous [rows, dim]
void gate_mul_fwd(const void* x, const void* gate, void* out, int64_t rows, int dim, int64_t xs, int64_t gs, int mode,
                  cudaStream_t stream) {
  const int64_t total = rows * (dim / 8);
  if (total == 0) return;
  const int g = grid_for(total);
  if (mode == 0)
    gate_mul_fwd_kernel<0><<<g, 256, 0, stream>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)gate, (__nv_bfloat16*)out, rows, dim, xs, gs);
  else
    gate_mul_fwd_kernel<1><<<g, 256, 0, stream>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)gate, (__nv_bfloat16*)out, rows, dim, xs, gs);
}

void gate_mul_bwd(const void* x, const void* gate, const void* dout, void* dx, void* dgate, int64_t rows, int dim,
                  int64_t xs, int64_t gs, int mode, cudaStream_t stream) {
  const int64_t total = rows * (dim / 8);
  if (total == 0) return;
  const int g = grid_for(total);
  if (mode == 0)
    gate_mul_bwd_kernel<0><<<g, 256, 0, stream>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)gate, (const __nv_bfloat16*)dout,
                                                   (__nv_bfloat16*)dx, (__nv_bfloat16*)dgate, rows, dim, xs, gs);
  else
    gate_mul_bwd_kernel<1><<<g, 256, 0, stream>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)gate, (const __nv_bfloat16*)dout,
                                                   (__nv_bfloat16*)dx, (__nv_bfloat16*)dgate, rows, dim, xs, gs);
}

}  // namespace mt
