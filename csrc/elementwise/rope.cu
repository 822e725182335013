// Rotary position embedding applied in place on a [tokens, heads, head_dim] bf16 view (row pitch given, so the
// q / k column blocks of a fused QKV projection output can be rotated where they lie).
// cos/sin come from a cached fp32 table [max_pos, rot_dim/2] that already includes the attention factor.
// Pairing: half-rotation (i, i + rot/2) or interleaved (2i, 2i+1).  With interleave the table entry used for
// element e is e mod rot/2 (the duplicated [sin, sin] / [cos, cos] layout of the reference implementation).
// inverse = true applies the transposed rotation (the backward pass).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cstdint>
#include "../api.h"

namespace mt {
namespace {

__global__ void rope_kernel(__nv_bfloat16* __restrict__ x, const float* __restrict__ cos_t,
                            const float* __restrict__ sin_t, const int* __restrict__ positions, int64_t tokens,
                            int seq_len, int heads, int head_dim, int rot_dim, int64_t row_stride, int interleave,
                            int inverse) {
  const int half = rot_dim >> 1;
  const int64_t total = tokens * heads * half;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int i = (int)(idx % half);
    const int64_t th = idx / half;
    const int h = (int)(th % heads);
    const int64_t t = th / heads;
    const int pos = positions ? positions[t] : (int)(t % seq_len);
    __nv_bfloat16* base = x + t * row_stride + (int64_t)h * head_dim;
    int e0, e1;
    float c0, s0, c1, s1;
    if (interleave) {
      e0 = 2 * i;
      e1 = 2 * i + 1;
      c0 = cos_t[(int64_t)pos * half + (e0 % half)];
      s0 = sin_t[(int64_t)pos * half + (e0 % half)];
      c1 = cos_t[(int64_t)pos * half + (e1 % half)];
      s1 = sin_t[(int64_t)pos * half + (e1 % half)];
    } else {
      e0 = i;
      e1 = i + half;
      c0 = c1 = cos_t[(int64_t)pos * half + i];
      s0 = s1 = sin_t[(int64_t)pos * half + i];
    }
    const float a = __bfloat162float(base[e0]);
    const float b = __bfloat162float(base[e1]);
    float o0, o1;
    if (!inverse) {
      // out[e0] = a*c0 - b*s0 ; out[e1] = b*c1 + a*s1
      o0 = a * c0 - b * s0;
      o1 = b * c1 + a * s1;
    } else {
      // transpose of the map above: d_a = g0*c0 + g1*s1 ; d_b = g1*c1 - g0*s0
      o0 = a * c0 + b * s1;
      o1 = b * c1 - a * s0;
    }
    base[e0] = __float2bfloat16(o0);
    base[e1] = __float2bfloat16(o1);
  }
}

union Pack8 {
  uint4 u;
  __nv_bfloat16 h[8];
};

// Half-rotation fast path: one thread rotates 8 pairs (i .. i+7, i+half .. i+half+7) with 16-byte accesses, reading
// from `src` and writing to `dst` (which may be the same buffer); columns past rot_dim are copied when src != dst.
__global__ void rope_half_vec_kernel(const __nv_bfloat16* __restrict__ src, __nv_bfloat16* __restrict__ dst,
                                     const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                     const int* __restrict__ positions, int64_t tokens, int seq_len, int heads,
                                     int head_dim, int rot_dim, int64_t src_stride, int64_t dst_stride, int inverse) {
  const int half = rot_dim >> 1;
  const int vec_half = half >> 3;                    // 16-byte chunks per half
  const int tail_vecs = (head_dim - rot_dim) >> 3;   // untouched chunks per head
  const int per_head = vec_half + tail_vecs;
  const int64_t total = tokens * heads * per_head;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int c = (int)(idx % per_head);
    const int64_t th = idx / per_head;
    const int h = (int)(th % heads);
    const int64_t t = th / heads;
    const __nv_bfloat16* sb = src + t * src_stride + (int64_t)h * head_dim;
    __nv_bfloat16* db = dst + t * dst_stride + (int64_t)h * head_dim;
    if (c >= vec_half) {
      if (src != dst) {
        const int off = rot_dim + (c - vec_half) * 8;
        *reinterpret_cast<uint4*>(db + off) = *reinterpret_cast<const uint4*>(sb + off);
      }
      continue;
    }
    const int pos = positions ? positions[t] : (int)(t % seq_len);
    const float4* cp = reinterpret_cast<const float4*>(cos_t + (int64_t)pos * half + c * 8);
    const float4* sp = reinterpret_cast<const float4*>(sin_t + (int64_t)pos * half + c * 8);
    const float4 c0 = cp[0], c1 = cp[1], s0 = sp[0], s1 = sp[1];
    const float cs[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
    const float sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
    Pack8 a, b, oa, ob;
    a.u = *reinterpret_cast<const uint4*>(sb + c * 8);
    b.u = *reinterpret_cast<const uint4*>(sb + half + c * 8);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float x0 = __bfloat162float(a.h[j]), x1 = __bfloat162float(b.h[j]);
      const float sgn = inverse ? -sn[j] : sn[j];
      oa.h[j] = __float2bfloat16(x0 * cs[j] - x1 * sgn);
      ob.h[j] = __float2bfloat16(x1 * cs[j] + x0 * sgn);
    }
    *reinterpret_cast<uint4*>(db + c * 8) = oa.u;
    *reinterpret_cast<uint4*>(db + half + c * 8) = ob.u;
  }
}

}  // namespace

void rope_apply(const void* src, void* dst, const float* cos_t, const float* sin_t, const int* positions,
                int64_t tokens, int seq_len, int heads, int head_dim, int rot_dim, int64_t src_stride,
                int64_t dst_stride, bool inverse, cudaStream_t stream) {
  const int per_head = (rot_dim / 2) / 8 + (head_dim - rot_dim) / 8;
  const int64_t total = tokens * heads * per_head;
  if (total == 0) return;
  int64_t blocks = (total + 255) / 256;
  if (blocks > 148 * 32) blocks = 148 * 32;
  rope_half_vec_kernel<<<(int)blocks, 256, 0, stream>>>((const __nv_bfloat16*)src, (__nv_bfloat16*)dst, cos_t, sin_t,
                                                        positions, tokens, seq_len, heads, head_dim, rot_dim,
                                                        src_stride, dst_stride, inverse ? 1 : 0);
}

void rope_inplace(void* x, const float* cos_t, const float* sin_t, const int* positions, int64_t tokens, int seq_len,
                  int heads, int head_dim, int rot_dim, int64_t row_stride, bool interleave, bool inverse,
                  cudaStream_t stream) {
  const int64_t total = tokens * heads * (rot_dim / 2);
  if (total == 0) return;
  int64_t blocks = (total + 255) / 256;
  if (blocks > 148 * 32) blocks = 148 * 32;
  rope_kernel<<<(int)blocks, 256, 0, stream>>>((__nv_bfloat16*)x, cos_t, sin_t, positions, tokens, seq_len, heads,
                                               head_dim, rot_dim, row_stride, interleave ? 1 : 0, inverse ? 1 : 0);
}

}  // namespace mt
