// RMSNorm forward / backward (bf16 I/O, fp32 math), optional fused residual add.
// Numerics contract: y = bf16(x * rsqrt(mean(x^2) + eps)) * bf16(w)  (the normalised value is rounded to
// bf16 before it is scaled, and the product is rounded again).
// One warp per row, 16-byte vector accesses; the second pass over the row is served from L1.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cstdint>
#include "../api.h"
#include "rmsnorm_noalloc.h"
#include <atomic>
#include <cstdio>

namespace mt {
namespace {

constexpr int kWarpsPerBlock = 8;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

union Pack8 {
  uint4 u;
  __nv_bfloat16 h[8];
};

__global__ void __launch_bounds__(kWarpsPerBlock * 32)
rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
                   const float* __restrict__ w, __nv_bfloat16* __restrict__ y, __nv_bfloat16* __restrict__ res_out,
                   float* __restrict__ rstd_out, int64_t rows, int dim, float eps) {
  const int lane = threadIdx.x & 31;
  const int64_t warp_global = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  const int64_t warp_stride = (int64_t)gridDim.x * kWarpsPerBlock;
  const int nvec = dim >> 3;
  for (int64_t row = warp_global; row < rows; row += warp_stride) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + row * dim);
    const uint4* rr = res ? reinterpret_cast<const uint4*>(res + row * dim) : nullptr;
    uint4* ro = res_out ? reinterpret_cast<uint4*>(res_out + row * dim) : nullptr;
    float ss = 0.f;
    for (int i = lane; i < nvec; i += 32) {
      Pack8 a;
      a.u = xr[i];
      if (rr) {
        Pack8 b;
        b.u = rr[i];
#pragma unroll
        for (int j = 0; j < 8; ++j) a.h[j] = __float2bfloat16(__bfloat162float(a.h[j]) + __bfloat162float(b.h[j]));
        if (ro) ro[i] = a.u;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float f = __bfloat162float(a.h[j]);
        ss += f * f;
      }
    }
    ss = warp_sum(ss);
    const float rstd = rsqrtf(ss / dim + eps);
    if (lane == 0 && rstd_out) rstd_out[row] = rstd;
    // second pass: the summed row (when a residual was added) is re-read from res_out, else from x
    const uint4* src = (rr && ro) ? reinterpret_cast<const uint4*>(res_out + row * dim) : xr;
    __syncwarp();
    uint4* yr = reinterpret_cast<uint4*>(y + row * dim);
    for (int i = lane; i < nvec; i += 32) {
      Pack8 a;
      a.u = src[i];
      if (rr && !ro) {
        Pack8 b;
        b.u = rr[i];
#pragma unroll
        for (int j = 0; j < 8; ++j) a.h[j] = __float2bfloat16(__bfloat162float(a.h[j]) + __bfloat162float(b.h[j]));
      }
      const float4 w0 = reinterpret_cast<const float4*>(w)[2 * i];
      const float4 w1 = reinterpret_cast<const float4*>(w)[2 * i + 1];
      const float wv[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
      Pack8 o;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const __nv_bfloat16 n = __float2bfloat16(__bfloat162float(a.h[j]) * rstd);
        o.h[j] = __float2bfloat16(__bfloat162float(n) * __bfloat162float(__float2bfloat16(wv[j])));
      }
      yr[i] = o.u;
    }
  }
}

// dx = rstd * (g - xhat * mean(xhat . g)) with g = w * dy, xhat = x * rstd;  dw += dy * xhat (per block partial).
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ w, const float* __restrict__ rstd_in,
                   const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ dres,
                   __nv_bfloat16* __restrict__ dx, float* __restrict__ dw_partial, int64_t rows, int dim) {
  extern __shared__ float dw_s[];
  for (int i = threadIdx.x; i < dim; i += blockDim.x) dw_s[i] = 0.f;
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int64_t warp_global = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  const int64_t warp_stride = (int64_t)gridDim.x * kWarpsPerBlock;
  const int nvec = dim >> 3;
  for (int64_t row = warp_global; row < rows; row += warp_stride) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + row * dim);
    const uint4* gr = reinterpret_cast<const uint4*>(dy + row * dim);
    const float rstd = rstd_in[row];
    float dot = 0.f;
    for (int i = lane; i < nvec; i += 32) {
      Pack8 a, g;
      a.u = xr[i];
      g.u = gr[i];
      const float4 w0 = reinterpret_cast<const float4*>(w)[2 * i];
      const float4 w1 = reinterpret_cast<const float4*>(w)[2 * i + 1];
      const float wv[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float xh = __bfloat162float(a.h[j]) * rstd;
        const float gy = __bfloat162float(g.h[j]);
        dot += xh * gy * wv[j];
        atomicAdd(&dw_s[i * 8 + j], gy * xh);
      }
    }
    dot = warp_sum(dot) / dim;
    const uint4* dr = dres ? reinterpret_cast<const uint4*>(dres + row * dim) : nullptr;
    uint4* dxr = reinterpret_cast<uint4*>(dx + row * dim);
    for (int i = lane; i < nvec; i += 32) {
      Pack8 a, g, o;
      a.u = xr[i];
      g.u = gr[i];
      Pack8 r;
      if (dr) r.u = dr[i];
      const float4 w0 = reinterpret_cast<const float4*>(w)[2 * i];
      const float4 w1 = reinterpret_cast<const float4*>(w)[2 * i + 1];
      const float wv[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float xh = __bfloat162float(a.h[j]) * rstd;
        float d = rstd * (__bfloat162float(g.h[j]) * wv[j] - xh * dot);
        if (dr) d += __bfloat162float(r.h[j]);
        o.h[j] = __float2bfloat16(d);
      }
      dxr[i] = o.u;
    }
  }
  __syncthreads();
  float* out = dw_partial + (int64_t)blockIdx.x * dim;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) out[i] = dw_s[i];
}

// Register-resident variant for dim = VPL * 256: every lane owns VPL 16-byte chunks of the row, reads x and dy once,
// and keeps its slice of the weight gradient in registers across all rows the warp processes (no shared-memory
// atomics in the row loop); the slices are combined through shared memory once per block at the end.
template <int VPL>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
rmsnorm_bwd_reg_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ w,
                       const float* __restrict__ rstd_in, const __nv_bfloat16* __restrict__ dy,
                       const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx,
                       float* __restrict__ dw_partial, int64_t rows) {
  constexpr int dim = VPL * 256;
  extern __shared__ float dw_s[];
  for (int i = threadIdx.x; i < dim; i += blockDim.x) dw_s[i] = 0.f;
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int64_t warp_global = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  const int64_t warp_stride = (int64_t)gridDim.x * kWarpsPerBlock;
  float dw_r[VPL * 8];
#pragma unroll
  for (int i = 0; i < VPL * 8; ++i) dw_r[i] = 0.f;
  for (int64_t row = warp_global; row < rows; row += warp_stride) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + row * dim);
    const uint4* gr = reinterpret_cast<const uint4*>(dy + row * dim);
    const float rstd = rstd_in[row];
    Pack8 a[VPL], g[VPL];
#pragma unroll
    for (int v = 0; v < VPL; ++v) {
      a[v].u = xr[v * 32 + lane];
      g[v].u = gr[v * 32 + lane];
    }
    float dot = 0.f;
#pragma unroll
    for (int v = 0; v < VPL; ++v) {
      const float4 w0 = reinterpret_cast<const float4*>(w)[2 * (v * 32 + lane)];
      const float4 w1 = reinterpret_cast<const float4*>(w)[2 * (v * 32 + lane) + 1];
      const float wv[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float xh = __bfloat162float(a[v].h[j]) * rstd;
        const float gy = __bfloat162float(g[v].h[j]);
        dot += xh * gy * wv[j];
        dw_r[v * 8 + j] += gy * xh;
      }
    }
    dot = warp_sum(dot) / dim;
    const uint4* dr = dres ? reinterpret_cast<const uint4*>(dres + row * dim) : nullptr;
    uint4* dxr = reinterpret_cast<uint4*>(dx + row * dim);
#pragma unroll
    for (int v = 0; v < VPL; ++v) {
      const float4 w0 = reinterpret_cast<const float4*>(w)[2 * (v * 32 + lane)];
      const float4 w1 = reinterpret_cast<const float4*>(w)[2 * (v * 32 + lane) + 1];
      const float wv[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
      Pack8 r, o;
      if (dr) r.u = dr[v * 32 + lane];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float xh = __bfloat162float(a[v].h[j]) * rstd;
        float d = rstd * (__bfloat162float(g[v].h[j]) * wv[j] - xh * dot);
        if (dr) d += __bfloat162float(r.h[j]);
        o.h[j] = __float2bfloat16(d);
      }
      dxr[v * 32 + lane] = o.u;
    }
  }
#pragma unroll
  for (int v = 0; v < VPL; ++v)
#pragma unroll
    for (int j = 0; j < 8; ++j) atomicAdd(&dw_s[(v * 32 + lane) * 8 + j], dw_r[v * 8 + j]);
  __syncthreads();
  float* out = dw_partial + (int64_t)blockIdx.x * dim;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) out[i] = dw_s[i];
}

// Column-owner variant for dim = 8 * blockDim.x (dim a multiple of 256, at most 8192): a block walks rows R at a time,
// every thread owns the same 8 columns of every row, so its slice of the weight gradient stays in 8 registers with
// no atomics, 2R 16-byte loads per thread are in flight, and the register count stays low enough for several
// blocks per SM.  The per-row dot product is a block reduction (warp shuffle, then one shared-memory exchange per
// R rows, double-buffered so one __syncthreads per iteration suffices).
template <int R, int THREADS>
__global__ void __launch_bounds__(THREADS)
rmsnorm_bwd_col_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ w,
                       const float* __restrict__ rstd_in, const __nv_bfloat16* __restrict__ dy,
                       const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx,
                       float* __restrict__ dw_partial, int64_t rows, int dim) {
  __shared__ float part[2][R][32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int vec = threadIdx.x;  // this thread's 16-byte chunk of every row
  const float4 w0 = reinterpret_cast<const float4*>(w)[2 * vec];
  const float4 w1 = reinterpret_cast<const float4*>(w)[2 * vec + 1];
  const float wv[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
  float dw_r[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  const float inv_dim = 1.f / dim;
  const int vecs_per_row = dim >> 3;
  int it = 0;
  for (int64_t row0 = (int64_t)blockIdx.x * R; row0 < rows; row0 += (int64_t)gridDim.x * R, ++it) {
    Pack8 a[R], g[R];
    float rs[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int64_t row = row0 + r;
      if (row < rows) {
        a[r].u = reinterpret_cast<const uint4*>(x)[row * vecs_per_row + vec];
        g[r].u = reinterpret_cast<const uint4*>(dy)[row * vecs_per_row + vec];
        rs[r] = rstd_in[row];
      } else {
        a[r].u = make_uint4(0, 0, 0, 0);
        g[r].u = make_uint4(0, 0, 0, 0);
        rs[r] = 0.f;
      }
    }
    float dot[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      float d = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float xh = __bfloat162float(a[r].h[j]) * rs[r];
        const float gy = __bfloat162float(g[r].h[j]);
        d = fmaf(xh * gy, wv[j], d);
        dw_r[j] = fmaf(gy, xh, dw_r[j]);
      }
      d = warp_sum(d);
      if (lane == 0) part[it & 1][r][warp] = d;
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < R; ++r) {
      float d = lane < nwarps ? part[it & 1][r][lane] : 0.f;
      dot[r] = warp_sum(d) * inv_dim;
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int64_t row = row0 + r;
      if (row >= rows) continue;
      Pack8 rr, o;
      if (dres) rr.u = reinterpret_cast<const uint4*>(dres)[row * vecs_per_row + vec];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float xh = __bfloat162float(a[r].h[j]) * rs[r];
        float d = rs[r] * (__bfloat162float(g[r].h[j]) * wv[j] - xh * dot[r]);
        if (dres) d += __bfloat162float(rr.h[j]);
        o.h[j] = __float2bfloat16(d);
      }
      reinterpret_cast<uint4*>(dx)[row * vecs_per_row + vec] = o.u;
    }
  }
  float* out = dw_partial + (int64_t)blockIdx.x * dim + vec * 8;
  reinterpret_cast<float4*>(out)[0] = make_float4(dw_r[0], dw_r[1], dw_r[2], dw_r[3]);
  reinterpret_cast<float4*>(out)[1] = make_float4(dw_r[4], dw_r[5], dw_r[6], dw_r[7]);
}

__global__ void rmsnorm_bwd_reduce_kernel(const float* __restrict__ partial, int num_partials, int dim,
                                          float* __restrict__ dw, int accumulate) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= dim) return;
  float s = 0.f;
  for (int p = 0; p < num_partials; ++p) s += partial[(int64_t)p * dim + i];
  dw[i] = accumulate ? dw[i] + s : s;
}

}  // namespace

void rmsnorm_fwd(const void* x, const void* residual, const float* w, void* y, void* residual_out, float* rstd,
                 int64_t rows, int dim, float eps, cudaStream_t stream) {
  if (rows == 0) return;
  int64_t blocks = (rows + kWarpsPerBlock - 1) / kWarpsPerBlock;
  if (blocks > 148 * 16) blocks = 148 * 16;
  rmsnorm_fwd_kernel<<<(int)blocks, kWarpsPerBlock * 32, 0, stream>>>(
      (const __nv_bfloat16*)x, (const __nv_bfloat16*)residual, w, (__nv_bfloat16*)y, (__nv_bfloat16*)residual_out,
      rstd, rows, dim, eps);
}

void rmsnorm_bwd(const void* x, const float* w, const float* rstd, const void* dy, const void* dres, void* dx,
                 float* dw_partial, int num_partials, int64_t rows, int dim, cudaStream_t stream) {
  if (rows == 0) return;
  auto xb = (const __nv_bfloat16*)x;
  auto gb = (const __nv_bfloat16*)dy;
  auto rb = (const __nv_bfloat16*)dres;
  auto ob = (__nv_bfloat16*)dx;
  const int threads = kWarpsPerBlock * 32;
  const size_t smem = dim * sizeof(float);
  if (dim % 256 == 0 && dim >= 1024 && dim <= 4096)  // up to 512 threads: four rows in flight per thread
    rmsnorm_bwd_col_kernel<4, 512><<<num_partials, dim / 8, 0, stream>>>(xb, w, rstd, gb, rb, ob, dw_partial, rows, dim);
  else if (dim % 256 == 0 && dim > 4096 && dim <= 8192)
    rmsnorm_bwd_col_kernel<2, 1024><<<num_partials, dim / 8, 0, stream>>>(xb, w, rstd, gb, rb, ob, dw_partial, rows, dim);
  else if (dim == 1024) rmsnorm_bwd_reg_kernel<4><<<num_partials, threads, smem, stream>>>(xb, w, rstd, gb, rb, ob, dw_partial, rows);
  else if (dim == 512) rmsnorm_bwd_reg_kernel<2><<<num_partials, threads, smem, stream>>>(xb, w, rstd, gb, rb, ob, dw_partial, rows);
  else if (dim == 256) rmsnorm_bwd_reg_kernel<1><<<num_partials, threads, smem, stream>>>(xb, w, rstd, gb, rb, ob, dw_partial, rows);
  else rmsnorm_bwd_kernel<<<num_partials, threads, smem, stream>>>(xb, w, rstd, gb, rb, ob, dw_partial, rows, dim);
}

void rmsnorm_bwd_reduce(const float* dw_partial, int num_partials, int dim, float* dw, bool accumulate,
                        cudaStream_t stream) {
  rmsnorm_bwd_reduce_kernel<<<(dim + 255) / 256, 256, 0, stream>>>(dw_partial, num_partials, dim, dw,
                                                                   accumulate ? 1 : 0);
}

}  // namespace mt

// ---------------------------------------------------------------------------------------------------------------
// Allocation-free variant (see rmsnorm_noalloc.h).  The per-block partial sums live in this file-scope device
// array instead of caller-provided memory.  In host code the array's name is only a handle: the device address
// the kernels need is obtained with cudaGetSymbolAddress, once per device.
static __device__ __align__(256) float g_rmsnorm_partials[MT_RMSNORM_NOALLOC_PARTIALS * MT_RMSNORM_NOALLOC_MAX_DIM];

namespace {
constexpr int kMaxDevices = 64;
// Written once per device with the same value by whichever host thread gets there first; atomic so that first
// calls from several threads do not race on the slot (relaxed order suffices: the value itself is all that is read).
std::atomic<float*> g_partials_addr[kMaxDevices];

int fail(char* err, size_t err_len, int code, const char* msg) {
  if (err && err_len > 0) std::snprintf(err, err_len, "%s", msg);
  return code;
}
}  // namespace

extern "C" int mt_rmsnorm_bwd_noalloc(const void* x, const float* w, const float* rstd, const void* dy,
                                      const void* dres, void* dx, float* dw, int64_t rows, int dim,
                                      int accumulate_dw, cudaStream_t stream, char* err, size_t err_len) {
  if (!w || !dw || (rows > 0 && (!x || !rstd || !dy || !dx)))  // an empty [0, dim] operand may have no address
    return fail(err, err_len, 1, "mt_rmsnorm_bwd_noalloc: null pointer argument");
  if (dim <= 0 || dim % 8 != 0) return fail(err, err_len, 2, "mt_rmsnorm_bwd_noalloc: dim must be a positive multiple of 8");
  if (dim > MT_RMSNORM_NOALLOC_MAX_DIM) {
    char msg[160];
    std::snprintf(msg, sizeof(msg), "mt_rmsnorm_bwd_noalloc: dim %d exceeds the built-in scratch limit of %d", dim,
                  MT_RMSNORM_NOALLOC_MAX_DIM);
    return fail(err, err_len, 3, msg);
  }
  if (rows < 0) return fail(err, err_len, 4, "mt_rmsnorm_bwd_noalloc: negative row count");
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(err, err_len, 5, cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices) return fail(err, err_len, 6, "mt_rmsnorm_bwd_noalloc: device index out of range");
  float* partials = g_partials_addr[dev].load(std::memory_order_relaxed);
  if (partials == nullptr) {  // one-time set-up for this device (current device = dev)
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_rmsnorm_partials);
    if (e != cudaSuccess) return fail(err, err_len, 7, cudaGetErrorString(e));
    partials = static_cast<float*>(p);
    g_partials_addr[dev].store(partials, std::memory_order_relaxed);
  }
  if (rows == 0) {
    // a sum over no rows: dw is zero (or left as it is when accumulating); reducing zero partial rows writes that
    mt::rmsnorm_bwd_reduce(partials, 0, dim, dw, accumulate_dw != 0, stream);
    e = cudaGetLastError();
    if (e != cudaSuccess) return fail(err, err_len, 8, cudaGetErrorString(e));
    return 0;
  }
  // same kernel selection as the ordinary entry point (bit-identical dx), with the built-in partial-sum array
  mt::rmsnorm_bwd(x, w, rstd, dy, dres, dx, partials, MT_RMSNORM_NOALLOC_PARTIALS, rows, dim, stream);
  mt::rmsnorm_bwd_reduce(partials, MT_RMSNORM_NOALLOC_PARTIALS, dim, dw, accumulate_dw != 0, stream);
  e = cudaGetLastError();
  if (e != cudaSuccess) return fail(err, err_len, 8, cudaGetErrorString(e));
  return 0;
}
