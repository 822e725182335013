// Chunk-parallel stage of the chunked Gated Delta Rule (forward and backward), fp32, one CTA per (batch, head, chunk).
//
// For a chunk of L = 64 tokens (mintext/modules/linear_attention.py:49-205) with raw queries / keys q, k [L, dk],
// values v [L, dv], write strengths beta [L] and log-decays g [L]:
//     qn = l2norm(q) / sqrt(dk)      kn = l2norm(k)      G = cumsum(g)      decay[i,j] = exp(G_i - G_j)  (j <= i)
//     A[i,j] = -beta_i <kn_i, kn_j> decay[i,j]  (j < i)          T = (I - A)^-1   (unit lower triangular)
//     U = T (beta v)       W = T (beta e^G kn)       M[i,j] = <qn_i, kn_j> decay[i,j]  (j <= i)
//     QG = qn e^G          KD = kn e^{G_L - G}       GL = e^{G_L}
// which are the operands the state-recurrence kernels (gdn_scan.cu) walk over.  Everything lives in shared memory:
// the 64x64 products run as register-tiled fp32 FMA loops (a thread owns a 4x4 or 4x8 block of the output, operands
// are read as float4 along the contraction or the output columns from padded tiles), T comes from inverting the
// four 16x16 diagonal blocks by forward substitution (one thread per column, in registers) followed by three
// block-row updates.  The forward saves T; the backward recomputes the cheap parts (normalisation, decays, the two
// Gram matrices) and propagates dW, dU, dQG, dM, dKD, dGL to dq, dk, dv, dbeta, dg:
//     dT = dU (beta v)^T + dW (beta e^G kn)^T        dA = T^T dT T^T  (strictly lower)
// and the product / exponent / normalisation rules of the definitions above; the gradient of the cumulative sum is a
// reverse cumulative sum inside the chunk.  Rows past the sequence end (last chunk) behave as zero inputs.
#include <cuda_runtime.h>
#include <cstdint>
#include <stdexcept>
#include "../api.h"

namespace mt {
namespace {

constexpr int L = 64;
constexpr int kThreads = 256;
constexpr int LDL = L + 4;  // leading dimension of the 64x64 tiles (bank-conflict-free float4 rows)
constexpr float kClamp = 30.f;

__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ void st4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ float clampf(float x) { return fminf(fmaxf(x, -kClamp), kClamp); }
__device__ __forceinline__ float inside(float x) { return (x > -kClamp && x < kClamp) ? 1.f : 0.f; }
// sum over the 16 threads that share an output row block (same threadIdx.x >> 4)
__device__ __forceinline__ float row_sum16(float v) {
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Thread layout of every product: ty = tid / 16 owns output rows 4 ty .. 4 ty + 3.
//   "nt" outputs (64 wide): columns tx + 16 c, c < 4.      "nn" / "tn" outputs (64 NC wide): columns 4 tx + 64 c + e.

// acc[r][c] += sum_k A[4ty+r][k] * B[tx+16c][k]
template <int K>
__device__ __forceinline__ void mm_nt(const float* __restrict__ A, int lda, const float* __restrict__ B, int ldb,
                                      float (&acc)[4][4]) {
  const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
#pragma unroll 2
  for (int k = 0; k < K; k += 4) {
    float4 a[4], b[4];
#pragma unroll
    for (int r = 0; r < 4; ++r) a[r] = ld4(A + (ty * 4 + r) * lda + k);
#pragma unroll
    for (int c = 0; c < 4; ++c) b[c] = ld4(B + (tx + 16 * c) * ldb + k);
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
      for (int c = 0; c < 4; ++c)
        acc[r][c] = fmaf(a[r].x, b[c].x, fmaf(a[r].y, b[c].y, fmaf(a[r].z, b[c].z, fmaf(a[r].w, b[c].w, acc[r][c]))));
  }
}

// acc[r][4c+e] += sum_{k in [kbeg, kend)} A[4ty+r][k] * B[k][4tx+64c+e]      (kbeg, kend multiples of 4)
template <int NC>
__device__ __forceinline__ void mm_nn(const float* __restrict__ A, int lda, const float* __restrict__ B, int ldb, int kbeg,
                                      int kend, float (&acc)[4][NC * 4]) {
  const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
  for (int k = kbeg; k < kend; k += 4) {
    float a[4][4];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const float4 t = ld4(A + (ty * 4 + r) * lda + k);
      a[r][0] = t.x, a[r][1] = t.y, a[r][2] = t.z, a[r][3] = t.w;
    }
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      float4 b[NC];
#pragma unroll
      for (int c = 0; c < NC; ++c) b[c] = ld4(B + (k + kk) * ldb + tx * 4 + 64 * c);
#pragma unroll
      for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int c = 0; c < NC; ++c) {
          acc[r][4 * c + 0] = fmaf(a[r][kk], b[c].x, acc[r][4 * c + 0]);
          acc[r][4 * c + 1] = fmaf(a[r][kk], b[c].y, acc[r][4 * c + 1]);
          acc[r][4 * c + 2] = fmaf(a[r][kk], b[c].z, acc[r][4 * c + 2]);
          acc[r][4 * c + 3] = fmaf(a[r][kk], b[c].w, acc[r][4 * c + 3]);
        }
    }
  }
}

// acc[r][4c+e] += sum_{k in [kbeg, kend)} A[k][4ty+r] * B[k][4tx+64c+e]
template <int NC>
__device__ __forceinline__ void mm_tn(const float* __restrict__ A, int lda, const float* __restrict__ B, int ldb, int kbeg,
                                      int kend, float (&acc)[4][NC * 4]) {
  const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
#pragma unroll 4
  for (int k = kbeg; k < kend; ++k) {
    const float4 t = ld4(A + k * lda + ty * 4);
    const float a[4] = {t.x, t.y, t.z, t.w};
    float4 b[NC];
#pragma unroll
    for (int c = 0; c < NC; ++c) b[c] = ld4(B + k * ldb + tx * 4 + 64 * c);
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
      for (int c = 0; c < NC; ++c) {
        acc[r][4 * c + 0] = fmaf(a[r], b[c].x, acc[r][4 * c + 0]);
        acc[r][4 * c + 1] = fmaf(a[r], b[c].y, acc[r][4 * c + 1]);
        acc[r][4 * c + 2] = fmaf(a[r], b[c].z, acc[r][4 * c + 2]);
        acc[r][4 * c + 3] = fmaf(a[r], b[c].w, acc[r][4 * c + 3]);
      }
  }
}

template <int N>
__device__ __forceinline__ void zero_acc(float (&acc)[4][N]) {
#pragma unroll
  for (int r = 0; r < 4; ++r)
#pragma unroll
    for (int c = 0; c < N; ++c) acc[r][c] = 0.f;
}

// rows [0, rows_valid) x columns [0, w) of a row-strided global tile -> shared tile [64][ld]; the rest (up to wp) zero
__device__ __forceinline__ void load_rows(float* dst, int ld, const float* __restrict__ src, int64_t row_stride, int w,
                                          int wp, int rows_valid) {
  const int per_row = wp / 4;
  for (int idx = threadIdx.x; idx < L * per_row; idx += kThreads) {
    const int r = idx / per_row, c = (idx % per_row) * 4;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (r < rows_valid && c < w) v = ld4(src + r * row_stride + c);
    st4(dst + r * ld + c, v);
  }
}

// Loads q and k rows, L2-normalises them (q also times dk^-0.5) into qn / kn and records the reciprocal norms;
// loads beta; cumulative log-decay G and e^G.  Ends with a __syncthreads().
template <int DK>
__device__ __forceinline__ void load_normalise(const GdnStrided& q, const GdnStrided& k, const GdnStrided& beta,
                                               const GdnStrided& g, int b, int h, int s0, int valid, float* qn, int ldq,
                                               float* kn, int ldk, float* bet, float* Gs, float* eGs, float* rqs,
                                               float* rks) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float* qp = q.p + b * q.sb + h * q.sh + (int64_t)s0 * q.ss;
  const float* kp = k.p + b * k.sb + h * k.sh + (int64_t)s0 * k.ss;
  constexpr float scale = DK == 64 ? 0.125f : 0.08838834764831845f;  // dk^-0.5
#pragma unroll 2
  for (int rr = 0; rr < 8; ++rr) {
    const int row = warp * 8 + rr;
    float4 x = make_float4(0.f, 0.f, 0.f, 0.f), y = x;
    if (row < valid && lane * 4 < DK) {
      x = ld4(qp + row * q.ss + lane * 4);
      y = ld4(kp + row * k.ss + lane * 4);
    }
    float sx = x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w, sy = y.x * y.x + y.y * y.y + y.z * y.z + y.w * y.w;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      sx += __shfl_xor_sync(0xffffffffu, sx, o);
      sy += __shfl_xor_sync(0xffffffffu, sy, o);
    }
    const float rq = rsqrtf(sx + 1e-6f), rk = rsqrtf(sy + 1e-6f), rqs_ = rq * scale;
    if (lane * 4 < DK) {
      st4(qn + row * ldq + lane * 4, make_float4(x.x * rqs_, x.y * rqs_, x.z * rqs_, x.w * rqs_));
      st4(kn + row * ldk + lane * 4, make_float4(y.x * rk, y.y * rk, y.z * rk, y.w * rk));
    }
    if (lane == 0 && rqs != nullptr) {
      rqs[row] = rq;
      rks[row] = rk;
    }
  }
  if (warp == 0) {
    const float* gp = g.p + b * g.sb + h * g.sh + (int64_t)s0 * g.ss;
    const float g0 = (2 * lane < valid) ? gp[(2 * lane) * g.ss] : 0.f;
    const float g1 = (2 * lane + 1 < valid) ? gp[(2 * lane + 1) * g.ss] : 0.f;
    float s = g0 + g1;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float t = __shfl_up_sync(0xffffffffu, s, o);
      if (lane >= o) s += t;
    }
    Gs[2 * lane] = s - g1;
    Gs[2 * lane + 1] = s;
    eGs[2 * lane] = __expf(clampf(s - g1));
    eGs[2 * lane + 1] = __expf(clampf(s));
  } else if (warp == 1) {
    const float* bp = beta.p + b * beta.sb + h * beta.sh + (int64_t)s0 * beta.ss;
    bet[lane] = lane < valid ? bp[lane * beta.ss] : 0.f;
    bet[lane + 32] = lane + 32 < valid ? bp[(lane + 32) * beta.ss] : 0.f;
  }
  __syncthreads();
}

// T = (I - A)^-1 for strictly lower triangular A [64][LDL] in shared memory; Rm: scratch of 16 x 52 floats.
__device__ __forceinline__ void invert_unit_lower(const float* Am, float* Tm, float* Rm) {
  const int tid = threadIdx.x;
  if (tid < 64) {
    const int b = tid >> 4, col = tid & 15;
    float d[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      float s = (i == col) ? 1.f : 0.f;
#pragma unroll
      for (int j = 0; j < i; ++j) s = fmaf(Am[(16 * b + i) * LDL + 16 * b + j], d[j], s);
      d[i] = s;
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) Tm[(16 * b + i) * LDL + 16 * b + col] = d[i];
  } else {
    // the six 16x16 blocks above the diagonal are zero
    for (int e = tid - 64; e < 6 * 256; e += kThreads - 64) {
      const int blk = e >> 8, i = (e >> 4) & 15, j = e & 15;
      const int bi = blk < 3 ? 0 : (blk < 5 ? 1 : 2);
      const int bj = blk < 3 ? blk + 1 : (blk < 5 ? blk - 1 : 3);
      Tm[(16 * bi + i) * LDL + 16 * bj + j] = 0.f;
    }
  }
  __syncthreads();
  for (int b = 1; b < 4; ++b) {
    const int nb = 16 * b;
    // R = A[block row b, 0:nb] T[0:nb, 0:nb]
    for (int e = tid; e < 16 * nb; e += kThreads) {
      const int i = e / nb, j = e % nb;
      float s = 0.f;
      for (int m = j; m < nb; ++m) s = fmaf(Am[(nb + i) * LDL + m], Tm[m * LDL + j], s);
      Rm[i * 52 + j] = s;
    }
    __syncthreads();
    // T[block row b, 0:nb] = D_b R
    for (int e = tid; e < 16 * nb; e += kThreads) {
      const int i = e / nb, j = e % nb;
      float s = 0.f;
#pragma unroll
      for (int m = 0; m < 16; ++m) s = fmaf(Tm[(nb + i) * LDL + nb + m], Rm[m * 52 + j], s);
      Tm[(nb + i) * LDL + j] = s;
    }
    __syncthreads();
  }
}

template <int DK, int DVP>
struct Smem {
  static constexpr int LDK = DK + 4, LDV = DVP + 4, LDB = LDK > LDV ? LDK : LDV;
  static constexpr int kVec = 9 * 64;  // beta, G, e^G, 1/|q|, 1/|k|, dbeta, dG, column sums, chunk-end term
  static constexpr size_t fwd_bytes = sizeof(float) * (size_t)(L * LDK + L * LDB + 2 * L * LDL + 16 * 52 + kVec);
  static constexpr size_t bwd_bytes = sizeof(float) * (size_t)(2 * L * LDK + 3 * L * LDL + 2 * L * LDB + kVec);
};

template <int DK, int DVP>
__global__ void __launch_bounds__(kThreads)
gdn_prep_fwd_kernel(GdnStrided q, GdnStrided k, GdnStrided v, GdnStrided beta, GdnStrided g, float* __restrict__ W,
                    float* __restrict__ U, float* __restrict__ QG, float* __restrict__ M, float* __restrict__ KD,
                    float* __restrict__ GL, float* __restrict__ Tsave, int H, int S, int C, int dv) {
  using SM = Smem<DK, DVP>;
  constexpr int LDK = SM::LDK, LDV = SM::LDV, LDB = SM::LDB;
  extern __shared__ __align__(16) float sh[];
  float* kn = sh;
  float* qb = kn + L * LDK;       // qn, later beta*v, later beta*e^G*kn
  float* Am = qb + L * LDB;
  float* Tm = Am + L * LDL;
  float* Rm = Tm + L * LDL;
  float* bet = Rm + 16 * 52;
  float* Gs = bet + 64;
  float* eGs = Gs + 64;
  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  const int64_t cb = blockIdx.x;
  const int bh = (int)(cb / C), c = (int)(cb % C), b = bh / H, h = bh % H;
  const int s0 = c * L, valid = min(L, S - s0);
  load_normalise<DK>(q, k, beta, g, b, h, s0, valid, qb, LDB, kn, LDK, bet, Gs, eGs, nullptr, nullptr);

  float acc[4][4];
  // A = -beta_i <kn_i, kn_j> decay, strictly lower
  zero_acc(acc);
  mm_nt<DK>(kn, LDK, kn, LDK, acc);
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int i = ty * 4 + r;
#pragma unroll
    for (int cc = 0; cc < 4; ++cc) {
      const int j = tx + 16 * cc;
      Am[i * LDL + j] = j < i ? -bet[i] * acc[r][cc] * __expf(clampf(Gs[i] - Gs[j])) : 0.f;
    }
  }
  // M = <qn_i, kn_j> decay, lower including the diagonal
  zero_acc(acc);
  mm_nt<DK>(qb, LDB, kn, LDK, acc);
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int i = ty * 4 + r;
#pragma unroll
    for (int cc = 0; cc < 4; ++cc) {
      const int j = tx + 16 * cc;
      M[cb * (L * L) + i * L + j] = j <= i ? acc[r][cc] * __expf(clampf(Gs[i] - Gs[j])) : 0.f;
    }
  }
  // QG, KD, GL
  {
    const float gl = Gs[L - 1];
    for (int idx = tid; idx < L * (DK / 4); idx += kThreads) {
      const int r = idx / (DK / 4), c4 = (idx % (DK / 4)) * 4;
      const float e = eGs[r], d = __expf(clampf(gl - Gs[r]));
      const float4 x = ld4(qb + r * LDB + c4), y = ld4(kn + r * LDK + c4);
      st4(QG + cb * (L * DK) + r * DK + c4, make_float4(x.x * e, x.y * e, x.z * e, x.w * e));
      st4(KD + cb * (L * DK) + r * DK + c4, make_float4(y.x * d, y.y * d, y.z * d, y.w * d));
    }
    if (tid == 0) GL[cb] = eGs[L - 1];
  }
  __syncthreads();
  invert_unit_lower(Am, Tm, Rm);
  for (int idx = tid; idx < L * (L / 4); idx += kThreads) {
    const int r = idx / (L / 4), c4 = (idx % (L / 4)) * 4;
    st4(Tsave + cb * (L * L) + r * L + c4, ld4(Tm + r * LDL + c4));
  }
  // U = T (beta v)
  {
    const float* vp = v.p + b * v.sb + h * v.sh + (int64_t)s0 * v.ss;
    load_rows(qb, LDV, vp, v.ss, dv, DVP, valid);
    __syncthreads();
    for (int idx = tid; idx < L * (DVP / 4); idx += kThreads) {
      const int r = idx / (DVP / 4), c4 = (idx % (DVP / 4)) * 4;
      const float bb = bet[r];
      float4 x = ld4(qb + r * LDV + c4);
      st4(qb + r * LDV + c4, make_float4(x.x * bb, x.y * bb, x.z * bb, x.w * bb));
    }
    __syncthreads();
    float au[4][DVP / 16];
    zero_acc(au);
    mm_nn<DVP / 64>(Tm, LDL, qb, LDV, 0, ty * 4 + 4, au);
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
      for (int cc = 0; cc < DVP / 64; ++cc) {
        const int col = tx * 4 + 64 * cc;
        if (col < dv)
          st4(U + (cb * L + ty * 4 + r) * dv + col, make_float4(au[r][4 * cc], au[r][4 * cc + 1], au[r][4 * cc + 2], au[r][4 * cc + 3]));
      }
    __syncthreads();
  }
  // W = T (beta e^G kn)
  {
    for (int idx = tid; idx < L * (DK / 4); idx += kThreads) {
      const int r = idx / (DK / 4), c4 = (idx % (DK / 4)) * 4;
      const float f = bet[r] * eGs[r];
      const float4 y = ld4(kn + r * LDK + c4);
      st4(qb + r * LDB + c4, make_float4(y.x * f, y.y * f, y.z * f, y.w * f));
    }
    __syncthreads();
    float aw[4][DK / 16];
    zero_acc(aw);
    mm_nn<DK / 64>(Tm, LDL, qb, LDB, 0, ty * 4 + 4, aw);
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
      for (int cc = 0; cc < DK / 64; ++cc)
        st4(W + (cb * L + ty * 4 + r) * DK + tx * 4 + 64 * cc,
            make_float4(aw[r][4 * cc], aw[r][4 * cc + 1], aw[r][4 * cc + 2], aw[r][4 * cc + 3]));
  }
}

template <int DK, int DVP>
__global__ void __launch_bounds__(kThreads)
gdn_prep_bwd_kernel(GdnStrided q, GdnStrided k, GdnStrided v, GdnStrided beta, GdnStrided g, const float* __restrict__ Tsave,
                    const float* __restrict__ dW, const float* __restrict__ dU, const float* __restrict__ dQG,
                    const float* __restrict__ dM, const float* __restrict__ dKD, const float* __restrict__ dGL,
                    float* __restrict__ dq, float* __restrict__ dk, float* __restrict__ dvo, float* __restrict__ dbeta,
                    float* __restrict__ dg, int H, int S, int C, int dv) {
  using SM = Smem<DK, DVP>;
  constexpr int LDK = SM::LDK, LDV = SM::LDV, LDB = SM::LDB;
  extern __shared__ __align__(16) float sh[];
  float* kn = sh;
  float* qn = kn + L * LDK;
  float* Tm = qn + L * LDK;
  float* Pm = Tm + L * LDL;   // dT, then dP
  float* Xm = Pm + L * LDL;   // T^T dT, then dQK
  float* b1 = Xm + L * LDL;   // dU, then dW
  float* b2 = b1 + L * LDB;   // v
  float* bet = b2 + L * LDB;
  float* Gs = bet + 64;
  float* eGs = Gs + 64;
  float* rqs = eGs + 64;
  float* rks = rqs + 64;
  float* dbs = rks + 64;      // dbeta
  float* dGs = dbs + 64;      // dG: row-side contributions
  float* dGc = dGs + 64;      // dG: column sums of E and the KD terms (subtracted)
  float* dGl = dGc + 64;      // dG of the chunk's last position from the KD terms (one float)
  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  const int64_t cb = blockIdx.x;
  const int bh = (int)(cb / C), c = (int)(cb % C), b = bh / H, h = bh % H;
  const int s0 = c * L, valid = min(L, S - s0);
  if (tid < 64) dbs[tid] = dGs[tid] = dGc[tid] = dGl[tid] = 0.f;
  for (int idx = tid; idx < L * (L / 4); idx += kThreads) {
    const int r = idx / (L / 4), c4 = (idx % (L / 4)) * 4;
    st4(Tm + r * LDL + c4, ld4(Tsave + cb * (L * L) + r * L + c4));
  }
  load_rows(b1, LDV, dU + cb * L * dv, dv, dv, DVP, L);
  {
    const float* vp = v.p + b * v.sb + h * v.sh + (int64_t)s0 * v.ss;
    load_rows(b2, LDV, vp, v.ss, dv, DVP, valid);
  }
  load_normalise<DK>(q, k, beta, g, b, h, s0, valid, qn, LDK, kn, LDK, bet, Gs, eGs, rqs, rks);  // ends with a barrier

  // ---- phase A: dT (value part) = dU v^T (column scale beta_j applied below); dBV = T^T dU -> dv, dbeta
  float accT[4][4];
  zero_acc(accT);
  mm_nt<DVP>(b1, LDV, b2, LDV, accT);
  {
    float av[4][DVP / 16];
    zero_acc(av);
    mm_tn<DVP / 64>(Tm, LDL, b1, LDV, ty * 4, L, av);
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int j = ty * 4 + r;
      const float bb = bet[j];
      float s = 0.f;
#pragma unroll
      for (int cc = 0; cc < DVP / 64; ++cc) {
        const int col = tx * 4 + 64 * cc;
        const float4 vv = ld4(b2 + j * LDV + col);
        s += av[r][4 * cc] * vv.x + av[r][4 * cc + 1] * vv.y + av[r][4 * cc + 2] * vv.z + av[r][4 * cc + 3] * vv.w;
        if (col < dv && j < valid)
          st4(dvo + ((int64_t)bh * S + s0 + j) * dv + col,
              make_float4(av[r][4 * cc] * bb, av[r][4 * cc + 1] * bb, av[r][4 * cc + 2] * bb, av[r][4 * cc + 3] * bb));
      }
      s = row_sum16(s);
      if (tx == 0) dbs[j] += s;
    }
  }
  __syncthreads();
  // ---- phase B: dT += dW (beta e^G kn)^T; dBK = T^T dW -> running dkn accumulator, dbeta, dG
  load_rows(b1, LDB, dW + cb * L * DK, DK, DK, DK, L);
  __syncthreads();
  float dkn[4][DK / 16];
  {
    float accT2[4][4];
    zero_acc(accT2);
    mm_nt<DK>(b1, LDB, kn, LDK, accT2);
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
      for (int cc = 0; cc < 4; ++cc) {
        const int j = tx + 16 * cc;
        Pm[(ty * 4 + r) * LDL + j] = bet[j] * (accT[r][cc] + eGs[j] * accT2[r][cc]);
      }
    zero_acc(dkn);
    mm_tn<DK / 64>(Tm, LDL, b1, LDB, ty * 4, L, dkn);
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int j = ty * 4 + r;
      float s = 0.f;
#pragma unroll
      for (int cc = 0; cc < DK / 64; ++cc) {
        const float4 kk = ld4(kn + j * LDK + tx * 4 + 64 * cc);
        s += dkn[r][4 * cc] * kk.x + dkn[r][4 * cc + 1] * kk.y + dkn[r][4 * cc + 2] * kk.z + dkn[r][4 * cc + 3] * kk.w;
      }
      s = row_sum16(s) * eGs[j];
      if (tx == 0) {
        dbs[j] += s;
        dGs[j] += bet[j] * s * inside(Gs[j]);
      }
      const float f = bet[j] * eGs[j];
#pragma unroll
      for (int e = 0; e < DK / 16; ++e) dkn[r][e] *= f;
    }
  }
  __syncthreads();
  // ---- phase C: dA = T^T dT T^T
  {
    float ax[4][4];
    zero_acc(ax);
    mm_tn<1>(Tm, LDL, Pm, LDL, ty * 4, L, ax);
#pragma unroll
    for (int r = 0; r < 4; ++r) st4(Xm + (ty * 4 + r) * LDL + tx * 4, make_float4(ax[r][0], ax[r][1], ax[r][2], ax[r][3]));
  }
  __syncthreads();
  float dA[4][4];
  zero_acc(dA);
  mm_nt<L>(Xm, LDL, Tm, LDL, dA);
  __syncthreads();  // Xm and Pm are rewritten below
  // ---- phase D: through A and M to the Gram matrices, beta and the decays
  {
    float P[4][4], QK[4][4];
    zero_acc(P);
    mm_nt<DK>(kn, LDK, kn, LDK, P);
    zero_acc(QK);
    mm_nt<DK>(qn, LDK, kn, LDK, QK);
    float csum[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int i = ty * 4 + r;
      const float bi = bet[i], gi = Gs[i];
      float sb = 0.f, se = 0.f;
#pragma unroll
      for (int cc = 0; cc < 4; ++cc) {
        const int j = tx + 16 * cc;
        const float diff = gi - Gs[j];
        const float dec = j <= i ? __expf(clampf(diff)) : 0.f;
        const float da = j < i ? dA[r][cc] : 0.f;
        const float dm = j <= i ? dM[cb * (L * L) + i * L + j] : 0.f;
        const float pda = P[r][cc] * dec * da;
        sb -= pda;
        const float e = (-bi * pda + dm * QK[r][cc] * dec) * inside(diff);
        se += e;
        csum[cc] += e;
        Pm[i * LDL + j] = -bi * dec * da;   // dP
        Xm[i * LDL + j] = dm * dec;         // dQK
      }
      sb = row_sum16(sb);
      se = row_sum16(se);
      if (tx == 0) {
        dbs[i] += sb;
        dGs[i] += se;
      }
    }
#pragma unroll
    for (int cc = 0; cc < 4; ++cc) atomicAdd(dGc + tx + 16 * cc, csum[cc]);
  }
  __syncthreads();
  // ---- phase E: dqn, dkn and the normalisations
  {
    float aq[4][DK / 16];
    zero_acc(aq);
    mm_nn<DK / 64>(Xm, LDL, kn, LDK, 0, ty * 4 + 4, aq);
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int i = ty * 4 + r;
      const float e = eGs[i];
      float sg = 0.f, sq = 0.f;
      float4 u[DK / 64];
#pragma unroll
      for (int cc = 0; cc < DK / 64; ++cc) {
        const int col = tx * 4 + 64 * cc;
        const float4 d = ld4(dQG + (cb * L + i) * DK + col);
        u[cc] = ld4(qn + i * LDK + col);
        sg += d.x * u[cc].x + d.y * u[cc].y + d.z * u[cc].z + d.w * u[cc].w;
        aq[r][4 * cc] += d.x * e, aq[r][4 * cc + 1] += d.y * e, aq[r][4 * cc + 2] += d.z * e, aq[r][4 * cc + 3] += d.w * e;
        sq += aq[r][4 * cc] * u[cc].x + aq[r][4 * cc + 1] * u[cc].y + aq[r][4 * cc + 2] * u[cc].z + aq[r][4 * cc + 3] * u[cc].w;
      }
      sg = row_sum16(sg);
      sq = row_sum16(sq);
      if (tx == 0) dGs[i] += sg * e * inside(Gs[i]);
      // qn = s rq q with s = dk^-0.5 and u = qn / s the unit vector:  dq = s rq (dqn - u <u, dqn>)
      constexpr float s = DK == 64 ? 0.125f : 0.08838834764831845f;
      const float rq = rqs[i];
      const float proj = sq / (s * s);   // qn proj = u <u, dqn>
      if (i < valid) {
#pragma unroll
        for (int cc = 0; cc < DK / 64; ++cc) {
          const int col = tx * 4 + 64 * cc;
          st4(dq + ((int64_t)bh * S + s0 + i) * DK + col,
              make_float4(s * rq * (aq[r][4 * cc] - u[cc].x * proj), s * rq * (aq[r][4 * cc + 1] - u[cc].y * proj),
                          s * rq * (aq[r][4 * cc + 2] - u[cc].z * proj), s * rq * (aq[r][4 * cc + 3] - u[cc].w * proj)));
        }
      }
    }
  }
  mm_tn<DK / 64>(Xm, LDL, qn, LDK, ty * 4, L, dkn);       // dQK^T qn
  mm_nn<DK / 64>(Pm, LDL, kn, LDK, 0, ty * 4 + 4, dkn);   // dP kn
  mm_tn<DK / 64>(Pm, LDL, kn, LDK, ty * 4, L, dkn);       // dP^T kn
  {
    const float gl = Gs[L - 1];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int j = ty * 4 + r;
      const float dl = gl - Gs[j], ekd = __expf(clampf(dl));
      float sk = 0.f, sp = 0.f;
      float4 u[DK / 64];
#pragma unroll
      for (int cc = 0; cc < DK / 64; ++cc) {
        const int col = tx * 4 + 64 * cc;
        const float4 d = ld4(dKD + (cb * L + j) * DK + col);
        u[cc] = ld4(kn + j * LDK + col);
        sk += d.x * u[cc].x + d.y * u[cc].y + d.z * u[cc].z + d.w * u[cc].w;
        dkn[r][4 * cc] += d.x * ekd, dkn[r][4 * cc + 1] += d.y * ekd, dkn[r][4 * cc + 2] += d.z * ekd, dkn[r][4 * cc + 3] += d.w * ekd;
        sp += dkn[r][4 * cc] * u[cc].x + dkn[r][4 * cc + 1] * u[cc].y + dkn[r][4 * cc + 2] * u[cc].z + dkn[r][4 * cc + 3] * u[cc].w;
      }
      sk = row_sum16(sk) * ekd * inside(dl);
      sp = row_sum16(sp);
      if (tx == 0) {
        atomicAdd(dGc + j, sk);          // dG_j -= sk
        atomicAdd(dGl, sk);              // dG_L += sk
      }
      const float rk = rks[j];
      if (j < valid) {
#pragma unroll
        for (int cc = 0; cc < DK / 64; ++cc) {
          const int col = tx * 4 + 64 * cc;
          st4(dk + ((int64_t)bh * S + s0 + j) * DK + col,
              make_float4(rk * (dkn[r][4 * cc] - u[cc].x * sp), rk * (dkn[r][4 * cc + 1] - u[cc].y * sp),
                          rk * (dkn[r][4 * cc + 2] - u[cc].z * sp), rk * (dkn[r][4 * cc + 3] - u[cc].w * sp)));
        }
      }
    }
  }
  __syncthreads();
  // ---- phase F: dg = reverse cumulative sum of dG; dbeta
  if (tid < 32) {
    const int lane = tid;
    float d0 = dGs[2 * lane] - dGc[2 * lane], d1 = dGs[2 * lane + 1] - dGc[2 * lane + 1];
    if (lane == 31) d1 += dGl[0] + dGL[cb] * eGs[L - 1] * inside(Gs[L - 1]);
    float s = d0 + d1;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float t = __shfl_down_sync(0xffffffffu, s, o);
      if (lane + o < 32) s += t;
    }
    // s = sum over elements 2 lane .. 63
    if (2 * lane < valid) dg[(int64_t)bh * S + s0 + 2 * lane] = s;
    if (2 * lane + 1 < valid) dg[(int64_t)bh * S + s0 + 2 * lane + 1] = s - d0;
  } else if (tid < 96) {
    const int i = tid - 32;
    if (i < valid) dbeta[(int64_t)bh * S + s0 + i] = dbs[i];
  }
}

template <int DK, int DVP>
void launch_fwd(const GdnStrided& q, const GdnStrided& k, const GdnStrided& v, const GdnStrided& beta, const GdnStrided& g,
                float* W, float* U, float* QG, float* M, float* KD, float* GL, float* T, int BH, int H, int S, int C, int dv,
                cudaStream_t stream) {
  auto kern = gdn_prep_fwd_kernel<DK, DVP>;
  constexpr size_t smem = Smem<DK, DVP>::fwd_bytes;
  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    configured = true;
  }
  kern<<<(unsigned)(BH * C), kThreads, smem, stream>>>(q, k, v, beta, g, W, U, QG, M, KD, GL, T, H, S, C, dv);
}

template <int DK, int DVP>
void launch_bwd(const GdnStrided& q, const GdnStrided& k, const GdnStrided& v, const GdnStrided& beta, const GdnStrided& g,
                const float* T, const float* dW, const float* dU, const float* dQG, const float* dM, const float* dKD,
                const float* dGL, float* dq, float* dk, float* dv_, float* dbeta, float* dg, int BH, int H, int S, int C, int dv,
                cudaStream_t stream) {
  auto kern = gdn_prep_bwd_kernel<DK, DVP>;
  constexpr size_t smem = Smem<DK, DVP>::bwd_bytes;
  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    configured = true;
  }
  kern<<<(unsigned)(BH * C), kThreads, smem, stream>>>(q, k, v, beta, g, T, dW, dU, dQG, dM, dKD, dGL, dq, dk, dv_, dbeta, dg, H,
                                                      S, C, dv);
}

}  // namespace

bool gdn_prep_supported(int dk, int dv) { return (dk == 64 || dk == 128) && dv % 32 == 0 && dv > 0 && dv <= 128; }

#define MT_GDN_DISPATCH(FN, ...)                                            \
  do {                                                                      \
    if (dk == 64 && dv <= 64) FN<64, 64>(__VA_ARGS__);                      \
    else if (dk == 64) FN<64, 128>(__VA_ARGS__);                            \
    else if (dv <= 64) FN<128, 64>(__VA_ARGS__);                            \
    else FN<128, 128>(__VA_ARGS__);                                         \
  } while (0)

void gdn_prep_fwd(const GdnStrided& q, const GdnStrided& k, const GdnStrided& v, const GdnStrided& beta, const GdnStrided& g,
                  float* W, float* U, float* QG, float* M, float* KD, float* GL, float* T, int B, int H, int S, int dk, int dv,
                  cudaStream_t stream) {
  if (!gdn_prep_supported(dk, dv)) throw std::runtime_error("gdn_prep: key dim must be 64 or 128, value dim a multiple of 32 up to 128");
  const int C = (S + L - 1) / L, BH = B * H;
  if (BH == 0 || C == 0) return;
  MT_GDN_DISPATCH(launch_fwd, q, k, v, beta, g, W, U, QG, M, KD, GL, T, BH, H, S, C, dv, stream);
}

void gdn_prep_bwd(const GdnStrided& q, const GdnStrided& k, const GdnStrided& v, const GdnStrided& beta, const GdnStrided& g,
                  const float* T, const float* dW, const float* dU, const float* dQG, const float* dM, const float* dKD,
                  const float* dGL, float* dq, float* dk_, float* dv_, float* dbeta, float* dg, int B, int H, int S, int dk,
                  int dv, cudaStream_t stream) {
  if (!gdn_prep_supported(dk, dv)) throw std::runtime_error("gdn_prep: key dim must be 64 or 128, value dim a multiple of 32 up to 128");
  const int C = (S + L - 1) / L, BH = B * H;
  if (BH == 0 || C == 0) return;
  MT_GDN_DISPATCH(launch_bwd, q, k, v, beta, g, T, dW, dU, dQG, dM, dKD, dGL, dq, dk_, dv_, dbeta, dg, BH, H, S, C, dv, stream);
}

}  // namespace mt
