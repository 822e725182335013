// Fused AdamW over a flat parameter shard plus the sum-of-squares reduction used for global-norm clipping.
// One pass reads grad (fp32 or bf16), m, v, master and writes m, v, master and the bf16 compute copy, so the
// separate fp32->bf16 weight cast of a mixed-precision step disappears.  Update rule (optax.adamw semantics):
//   m <- b1 m + (1-b1) g ; v <- b2 v + (1-b2) g^2 ; p <- p - lr * ( (m/bc1) / (sqrt(v/bc2) + eps) + wd * p )
// The square root and the division of the update are the IEEE-rounded intrinsics: the build's fast-math flag would
// otherwise turn them into approximations, and the optimizer is where an error repeats every step.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cstdint>
#include "../api.h"

namespace mt {
namespace {

template <bool GRAD_F32>
__global__ void adamw_kernel(float* __restrict__ master, float* __restrict__ m, float* __restrict__ v,
                             const void* __restrict__ grad, __nv_bfloat16* __restrict__ pbf, int64_t n, float lr,
                             float b1, float b2, float eps, float wd, float bc1, float bc2, float grad_scale,
                             const float* __restrict__ clip_coef) {
  const float gs = clip_coef ? grad_scale * (*clip_coef) : grad_scale;
  const float rbc1 = __fdiv_rn(1.f, bc1), rbc2 = __fdiv_rn(1.f, bc2);
  const int64_t nvec = n >> 2;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (int64_t)gridDim.x * blockDim.x) {
    float g[4];
    if (GRAD_F32) {
      const float4 t = reinterpret_cast<const float4*>(grad)[i];
      g[0] = t.x; g[1] = t.y; g[2] = t.z; g[3] = t.w;
    } else {
      const uint2 t = reinterpret_cast<const uint2*>(grad)[i];
      const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&t.x);
      const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&t.y);
      g[0] = __low2float(a); g[1] = __high2float(a); g[2] = __low2float(b); g[3] = __high2float(b);
    }
    float4 mm = reinterpret_cast<float4*>(m)[i];
    float4 vv = reinterpret_cast<float4*>(v)[i];
    float4 pp = reinterpret_cast<float4*>(master)[i];
    float* mp = &mm.x; float* vp = &vv.x; float* ppp = &pp.x;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float gj = g[j] * gs;
      mp[j] = b1 * mp[j] + (1.f - b1) * gj;
      vp[j] = b2 * vp[j] + (1.f - b2) * gj * gj;
      const float upd = __fdiv_rn(mp[j] * rbc1, __fsqrt_rn(vp[j] * rbc2) + eps) + wd * ppp[j];
      ppp[j] -= lr * upd;
    }
    reinterpret_cast<float4*>(m)[i] = mm;
    reinterpret_cast<float4*>(v)[i] = vv;
    reinterpret_cast<float4*>(master)[i] = pp;
    if (pbf) {
      uint2 o;
      __nv_bfloat162 a = __floats2bfloat162_rn(pp.x, pp.y);
      __nv_bfloat162 b = __floats2bfloat162_rn(pp.z, pp.w);
      o.x = *reinterpret_cast<uint32_t*>(&a);
      o.y = *reinterpret_cast<uint32_t*>(&b);
      reinterpret_cast<uint2*>(pbf)[i] = o;
    }
  }
  // scalar tail
  for (int64_t i = (nvec << 2) + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x) {
    const float gj = (GRAD_F32 ? reinterpret_cast<const float*>(grad)[i]
                               : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(grad)[i])) * gs;
    const float mj = b1 * m[i] + (1.f - b1) * gj;
    const float vj = b2 * v[i] + (1.f - b2) * gj * gj;
    const float upd = __fdiv_rn(mj * rbc1, __fsqrt_rn(vj * rbc2) + eps) + wd * master[i];
    const float p = master[i] - lr * upd;
    m[i] = mj; v[i] = vj; master[i] = p;
    if (pbf) pbf[i] = __float2bfloat16(p);
  }
}

// Sum of squares.  A thread keeps four 16-byte loads in flight per iteration (the kernel is a pure read stream);
// the ragged tail (and a misaligned base) falls back to scalar loads.
template <bool F32>
__global__ void sumsq_kernel(const void* __restrict__ x, int64_t n, float* __restrict__ out) {
  constexpr int EPV = F32 ? 4 : 8;  // elements per 16-byte vector
  float s = 0.f;
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x, nthreads = (int64_t)gridDim.x * blockDim.x;
  const bool aligned = (reinterpret_cast<uintptr_t>(x) & 15) == 0;
  const int64_t nvec = aligned ? n / EPV : 0;
  const uint4* xv = reinterpret_cast<const uint4*>(x);
  auto add_vec = [&s](const uint4& v) {
    if (F32) {
      const float a = __uint_as_float(v.x), b = __uint_as_float(v.y), c = __uint_as_float(v.z), d = __uint_as_float(v.w);
      s += a * a + b * b + c * c + d * d;
    } else {
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float lo = __uint_as_float(w[j] << 16), hi = __uint_as_float(w[j] & 0xffff0000u);
        s += lo * lo + hi * hi;
      }
    }
  };
  int64_t i = tid;
  for (; i + 3 * nthreads < nvec; i += 4 * nthreads) {
    const uint4 v0 = xv[i], v1 = xv[i + nthreads], v2 = xv[i + 2 * nthreads], v3 = xv[i + 3 * nthreads];
    add_vec(v0);
    add_vec(v1);
    add_vec(v2);
    add_vec(v3);
  }
  for (; i < nvec; i += nthreads) add_vec(xv[i]);
  for (int64_t k = nvec * EPV + tid; k < n; k += nthreads) {
    const float f = F32 ? reinterpret_cast<const float*>(x)[k]
                        : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(x)[k]);
    s += f * f;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  __shared__ float red[32];
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x < 32) {
    s = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (threadIdx.x == 0) atomicAdd(out, s);
  }
}

inline int grid_for(int64_t total) {
  int64_t b = (total + 255) / 256;
  if (b < 1) b = 1;
  return (int)(b > 148 * 8 ? 148 * 8 : b);
}

}  // namespace

void adamw_step(float* master, float* m, float* v, const void* grad, bool grad_f32, void* param_bf16, int64_t n,
                float lr, float b1, float b2, float eps, float wd, float bc1, float bc2, float grad_scale,
                const float* clip_coef, cudaStream_t stream) {
  if (n == 0) return;
  const int g = grid_for(n / 4);
  if (grad_f32)
    adamw_kernel<true><<<g, 256, 0, stream>>>(master, m, v, grad, (__nv_bfloat16*)param_bf16, n, lr, b1, b2, eps, wd,
                                              bc1, bc2, grad_scale, clip_coef);
  else
    adamw_kernel<false><<<g, 256, 0, stream>>>(master, m, v, grad, (__nv_bfloat16*)param_bf16, n, lr, b1, b2, eps, wd,
                                               bc1, bc2, grad_scale, clip_coef);
}

void sumsq(const void* x, bool is_f32, int64_t n, float* out_accum, cudaStream_t stream) {
  if (n == 0) return;
  const int g = grid_for(n / 16 + 1);
  if (is_f32) sumsq_kernel<true><<<g, 256, 0, stream>>>(x, n, out_accum);
  else sumsq_kernel<false><<<g, 256, 0, stream>>>(x, n, out_accum);
}

}  // namespace mt
