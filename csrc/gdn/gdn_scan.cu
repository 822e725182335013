// Inter-chunk state recurrence of the chunked Gated Delta Rule (forward and backward), fp32.
//
// Per (batch, head) the chunked algorithm (mintext/modules/linear_attention.py:49-205) ends in a sequential walk over
// the chunks with a [dk, dv] state S:
//     V' = U - W S            O = QG S + M V'            S <- gl * S + KD^T V'
// where, per chunk of L = 64 tokens, W [L,dk] (decayed keys through the WY inverse), U [L,dv] (corrected values),
// QG [L,dk] (queries times cumulative decay), M [L,L] (masked decayed q k^T), KD [L,dk] (keys decayed to the chunk
// end) and gl (the chunk's total decay) are produced chunk-parallel beforehand.  The columns of S evolve
// independently, so one CTA owns 32 value columns of one (batch, head): grid (B*H, dv/32), the state slice lives in
// shared memory for the whole walk, every chunk's operands are staged in shared memory once and consumed by
// register-tiled fp32 FMA loops (256 threads; a warp shares the row operand by broadcast, lanes own columns).
// Forward also records the state at every chunk start for the backward walk, which runs the chunks in reverse with
// the state gradient dS in shared memory and produces dU directly and dW, dQG, dM, dKD, dgl by atomic adds (they
// sum over the dv/32 column slices).
#include <cuda_runtime.h>
#include <cstdint>
#include <stdexcept>
#include "../api.h"

namespace mt {
namespace {

constexpr int L = 64;      // chunk length
constexpr int DVB = 32;    // value columns per CTA
constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int SP = DVB + 1;  // padded row length of the state slices (conflict-free column and row access)
constexpr int VP = DVB + 1;  // same for the V', dV' and dO tiles

__device__ __forceinline__ void load_tile(float* dst, const float* __restrict__ src, int n) {
  for (int i = threadIdx.x * 4; i < n; i += kThreads * 4) *reinterpret_cast<float4*>(dst + i) = *reinterpret_cast<const float4*>(src + i);
}

// shared memory (floats): W[L*dk] QG[L*dk] KD[L*dk] M[L*L] U[L*DVB] V[L*DVB] S[dk*SP]  (+ backward extras)
template <int DK>
__global__ void __launch_bounds__(kThreads)
gdn_scan_fwd_kernel(const float* __restrict__ W, const float* __restrict__ U, const float* __restrict__ QG,
                    const float* __restrict__ M, const float* __restrict__ KD, const float* __restrict__ GL,
                    float* __restrict__ O, float* __restrict__ Sstart, int C, int dv) {
  extern __shared__ float sh[];
  float* w_s = sh;
  float* qg_s = w_s + L * DK;
  float* kd_s = qg_s + L * DK;
  float* m_s = kd_s + L * DK;
  float* u_s = m_s + L * L;
  float* v_s = u_s + L * DVB;
  float* s_s = v_s + L * VP;
  const int bh = blockIdx.x;
  const int j0 = blockIdx.y * DVB;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < DK * SP; i += kThreads) s_s[i] = 0.f;
  __syncthreads();
  for (int c = 0; c < C; ++c) {
    const int64_t cb = (int64_t)bh * C + c;
    load_tile(w_s, W + cb * L * DK, L * DK);
    load_tile(qg_s, QG + cb * L * DK, L * DK);
    load_tile(kd_s, KD + cb * L * DK, L * DK);
    load_tile(m_s, M + cb * L * L, L * L);
    for (int i = threadIdx.x; i < L * DVB; i += kThreads) u_s[i] = U[(cb * L + i / DVB) * dv + j0 + (i % DVB)];
    // the state at the chunk start, for the backward walk
    for (int i = threadIdx.x; i < DK * DVB; i += kThreads)
      Sstart[(cb * DK + i / DVB) * dv + j0 + (i % DVB)] = s_s[(i / DVB) * SP + (i % DVB)];
    __syncthreads();
    // V'[l, lane] = U - W S ; rows l = warp + 8 i
    float acc[L / kWarps], accq[L / kWarps];
#pragma unroll
    for (int i = 0; i < L / kWarps; ++i) acc[i] = accq[i] = 0.f;
    for (int k = 0; k < DK; k += 4) {
      const float s0 = s_s[(k + 0) * SP + lane], s1 = s_s[(k + 1) * SP + lane], s2 = s_s[(k + 2) * SP + lane],
                  s3 = s_s[(k + 3) * SP + lane];
#pragma unroll
      for (int i = 0; i < L / kWarps; ++i) {
        const int l = warp + kWarps * i;
        const float4 w4 = *reinterpret_cast<const float4*>(w_s + l * DK + k);
        const float4 q4 = *reinterpret_cast<const float4*>(qg_s + l * DK + k);
        acc[i] = fmaf(w4.x, s0, fmaf(w4.y, s1, fmaf(w4.z, s2, fmaf(w4.w, s3, acc[i]))));
        accq[i] = fmaf(q4.x, s0, fmaf(q4.y, s1, fmaf(q4.z, s2, fmaf(q4.w, s3, accq[i]))));
      }
    }
#pragma unroll
    for (int i = 0; i < L / kWarps; ++i) {
      const int l = warp + kWarps * i;
      v_s[l * VP + lane] = u_s[l * DVB + lane] - acc[i];
    }
    __syncthreads();
    // O[l, lane] = QG S + M V' : the warp's eight rows share every V' load (32 FMAs per 12 shared-memory loads)
    for (int m = 0; m < L; m += 4) {
      const float v0 = v_s[(m + 0) * VP + lane], v1 = v_s[(m + 1) * VP + lane], v2 = v_s[(m + 2) * VP + lane],
                  v3 = v_s[(m + 3) * VP + lane];
#pragma unroll
      for (int i = 0; i < L / kWarps; ++i) {
        const float4 m4 = *reinterpret_cast<const float4*>(m_s + (warp + kWarps * i) * L + m);
        accq[i] = fmaf(m4.x, v0, fmaf(m4.y, v1, fmaf(m4.z, v2, fmaf(m4.w, v3, accq[i]))));
      }
    }
#pragma unroll
    for (int i = 0; i < L / kWarps; ++i) O[(cb * L + warp + kWarps * i) * dv + j0 + lane] = accq[i];
    // S[k, lane] = gl * S + sum_l KD[l, k] V'[l, lane] ; a warp owns DK / 8 adjacent key rows, so that one V' load
    // and DK / 32 vector loads of KD feed DK / 8 FMAs (each thread owns its own S entries)
    {
      constexpr int KW = DK / kWarps;
      const int k0 = warp * KW;
      const float gl = GL[cb];
      float a[KW];
#pragma unroll
      for (int i = 0; i < KW; ++i) a[i] = gl * s_s[(k0 + i) * SP + lane];
#pragma unroll 4
      for (int l = 0; l < L; ++l) {
        const float v = v_s[l * VP + lane];
#pragma unroll
        for (int i = 0; i < KW; i += 4) {
          const float4 k4 = *reinterpret_cast<const float4*>(kd_s + l * DK + k0 + i);
          a[i] = fmaf(k4.x, v, a[i]);
          a[i + 1] = fmaf(k4.y, v, a[i + 1]);
          a[i + 2] = fmaf(k4.z, v, a[i + 2]);
          a[i + 3] = fmaf(k4.w, v, a[i + 3]);
        }
      }
#pragma unroll
      for (int i = 0; i < KW; ++i) s_s[(k0 + i) * SP + lane] = a[i];
    }
    __syncthreads();
  }
}

// Backward walk.  Extra shared memory: dO[L*DVB] dV[L*DVB] Sc[dk*SP] (chunk-start state) dS[dk*SP].
template <int DK>
__global__ void __launch_bounds__(kThreads)
gdn_scan_bwd_kernel(const float* __restrict__ W, const float* __restrict__ U, const float* __restrict__ QG,
                    const float* __restrict__ M, const float* __restrict__ KD, const float* __restrict__ GL,
                    const float* __restrict__ Sstart, const float* __restrict__ dO, float* __restrict__ dW,
                    float* __restrict__ dU, float* __restrict__ dQG, float* __restrict__ dM, float* __restrict__ dKD,
                    float* __restrict__ dGL, int C, int dv) {
  extern __shared__ float sh[];
  float* w_s = sh;
  float* qg_s = w_s + L * DK;
  float* kd_s = qg_s + L * DK;
  float* m_s = kd_s + L * DK;
  float* u_s = m_s + L * L;
  float* v_s = u_s + L * DVB;     // V' (recomputed)
  float* do_s = v_s + L * VP;
  float* dv_s = do_s + L * VP;    // dV'
  float* sc_s = dv_s + L * VP;    // state at the chunk start
  float* ds_s = sc_s + DK * SP;   // gradient of the state after this chunk
  __shared__ float red[kWarps];
  const int bh = blockIdx.x;
  const int j0 = blockIdx.y * DVB;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < DK * SP; i += kThreads) ds_s[i] = 0.f;
  __syncthreads();
  for (int c = C - 1; c >= 0; --c) {
    const int64_t cb = (int64_t)bh * C + c;
    load_tile(w_s, W + cb * L * DK, L * DK);
    load_tile(qg_s, QG + cb * L * DK, L * DK);
    load_tile(kd_s, KD + cb * L * DK, L * DK);
    load_tile(m_s, M + cb * L * L, L * L);
    for (int i = threadIdx.x; i < L * DVB; i += kThreads) {
      const int64_t g = (cb * L + i / DVB) * dv + j0 + (i % DVB);
      u_s[i] = U[g];
      do_s[(i / DVB) * VP + (i % DVB)] = dO[g];
    }
    for (int i = threadIdx.x; i < DK * DVB; i += kThreads)
      sc_s[(i / DVB) * SP + (i % DVB)] = Sstart[(cb * DK + i / DVB) * dv + j0 + (i % DVB)];
    __syncthreads();
    const float gl = GL[cb];
    // (1) V'[l, lane] = U - W Sc       (2) part of dV': KD dS   -- both dots over k
    {
      float acc[L / kWarps], acd[L / kWarps];
#pragma unroll
      for (int i = 0; i < L / kWarps; ++i) acc[i] = acd[i] = 0.f;
      for (int k = 0; k < DK; k += 4) {
        float s[4], d[4];
#pragma unroll
        for (int x = 0; x < 4; ++x) {
          s[x] = sc_s[(k + x) * SP + lane];
          d[x] = ds_s[(k + x) * SP + lane];
        }
#pragma unroll
        for (int i = 0; i < L / kWarps; ++i) {
          const int l = warp + kWarps * i;
          const float4 w4 = *reinterpret_cast<const float4*>(w_s + l * DK + k);
          const float4 k4 = *reinterpret_cast<const float4*>(kd_s + l * DK + k);
          acc[i] = fmaf(w4.x, s[0], fmaf(w4.y, s[1], fmaf(w4.z, s[2], fmaf(w4.w, s[3], acc[i]))));
          acd[i] = fmaf(k4.x, d[0], fmaf(k4.y, d[1], fmaf(k4.z, d[2], fmaf(k4.w, d[3], acd[i]))));
        }
      }
#pragma unroll
      for (int i = 0; i < L / kWarps; ++i) {
        const int l = warp + kWarps * i;
        v_s[l * VP + lane] = u_s[l * DVB + lane] - acc[i];
        dv_s[l * VP + lane] = acd[i];
      }
    }
    __syncthreads();
    // (3) dV'[m, lane] += sum_l M[l, m] dO[l, lane] ; then dU = dV'.  A warp owns the eight adjacent rows
    //     m = 8 warp .. 8 warp + 7: one dO load and two vector loads of M feed eight FMAs.
    {
      const int m0 = warp * (L / kWarps);
      float a[L / kWarps];
#pragma unroll
      for (int i = 0; i < L / kWarps; ++i) a[i] = dv_s[(m0 + i) * VP + lane];
#pragma unroll 4
      for (int l = 0; l < L; ++l) {
        const float d = do_s[l * VP + lane];
        const float4 ma = *reinterpret_cast<const float4*>(m_s + l * L + m0);
        const float4 mb = *reinterpret_cast<const float4*>(m_s + l * L + m0 + 4);
        a[0] = fmaf(ma.x, d, a[0]); a[1] = fmaf(ma.y, d, a[1]); a[2] = fmaf(ma.z, d, a[2]); a[3] = fmaf(ma.w, d, a[3]);
        a[4] = fmaf(mb.x, d, a[4]); a[5] = fmaf(mb.y, d, a[5]); a[6] = fmaf(mb.z, d, a[6]); a[7] = fmaf(mb.w, d, a[7]);
      }
      __syncthreads();  // every warp has read the dV' rows it needs before any row changes
#pragma unroll
      for (int i = 0; i < L / kWarps; ++i) {
        dv_s[(m0 + i) * VP + lane] = a[i];
        dU[(cb * L + m0 + i) * dv + j0 + lane] = a[i];
      }
    }
    __syncthreads();
    // (4) outputs that reduce over this CTA's 32 columns; a thread owns the key rows k = lane + 32 x (all of them:
    //     conflict-free in the padded state tiles) and, per pass, four of its rows l = warp + 8 r; it walks the 32
    //     columns and then adds into global memory (the dv/32 column slices of a head all contribute):
    //     dQG[l,k] = <dO[l,:], Sc[k,:]>   dW[l,k] = -<dV'[l,:], Sc[k,:]>   dKD[l,k] = <V'[l,:], dS[k,:]>
    {
      constexpr int KX = DK / 32;
      for (int rp = 0; rp < L / kWarps; rp += 4) {
        float aq[4][KX], aw[4][KX], ak[4][KX];
#pragma unroll
        for (int r = 0; r < 4; ++r)
#pragma unroll
          for (int x = 0; x < KX; ++x) aq[r][x] = aw[r][x] = ak[r][x] = 0.f;
#pragma unroll 2
        for (int j = 0; j < DVB; ++j) {
          float sv[KX], dsv[KX];
#pragma unroll
          for (int x = 0; x < KX; ++x) {
            sv[x] = sc_s[(lane + 32 * x) * SP + j];
            dsv[x] = ds_s[(lane + 32 * x) * SP + j];
          }
#pragma unroll
          for (int r = 0; r < 4; ++r) {
            const int l = warp + kWarps * (rp + r);
            const float d = do_s[l * VP + j], g = dv_s[l * VP + j], v = v_s[l * VP + j];
#pragma unroll
            for (int x = 0; x < KX; ++x) {
              aq[r][x] = fmaf(d, sv[x], aq[r][x]);
              aw[r][x] = fmaf(g, sv[x], aw[r][x]);
              ak[r][x] = fmaf(v, dsv[x], ak[r][x]);
            }
          }
        }
#pragma unroll
        for (int r = 0; r < 4; ++r)
#pragma unroll
          for (int x = 0; x < KX; ++x) {
            const int64_t g = (cb * L + warp + kWarps * (rp + r)) * DK + lane + 32 * x;
            atomicAdd(dQG + g, aq[r][x]);
            atomicAdd(dW + g, -aw[r][x]);
            atomicAdd(dKD + g, ak[r][x]);
          }
      }
    }
    //     dM[l, m] = <dO[l,:], V'[m,:]>
    for (int x = 0; x < L / 32; ++x) {
      const int m = lane + 32 * x;
      float am[L / kWarps];
#pragma unroll
      for (int r = 0; r < L / kWarps; ++r) am[r] = 0.f;
      for (int j = 0; j < DVB; ++j) {
        const float vm = v_s[m * VP + j];
#pragma unroll
        for (int r = 0; r < L / kWarps; ++r) am[r] = fmaf(do_s[(warp + kWarps * r) * VP + j], vm, am[r]);
      }
#pragma unroll
      for (int r = 0; r < L / kWarps; ++r) atomicAdd(dM + (cb * L + warp + kWarps * r) * L + m, am[r]);
    }
    // (5) dgl = <dS, Sc>
    {
      float a = 0.f;
      for (int i = threadIdx.x; i < DK * DVB; i += kThreads) a += ds_s[(i / DVB) * SP + (i % DVB)] * sc_s[(i / DVB) * SP + (i % DVB)];
#pragma unroll
      for (int x = 16; x > 0; x >>= 1) a += __shfl_xor_sync(0xffffffffu, a, x);
      if (lane == 0) red[warp] = a;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      float a = 0.f;
      for (int w = 0; w < kWarps; ++w) a += red[w];
      atomicAdd(dGL + cb, a);
    }
    // (6) dS_prev[k, lane] = gl * dS + sum_l QG[l,k] dO[l,lane] - sum_l W[l,k] dV'[l,lane] ; a warp owns DK / 8
    //     adjacent key rows (two loads of dO / dV' and DK / 16 vector loads feed DK / 4 FMAs)
    {
      constexpr int KW = DK / kWarps;
      const int k0 = warp * KW;
      float a[KW];
#pragma unroll
      for (int i = 0; i < KW; ++i) a[i] = gl * ds_s[(k0 + i) * SP + lane];
#pragma unroll 2
      for (int l = 0; l < L; ++l) {
        const float d = do_s[l * VP + lane], g = -dv_s[l * VP + lane];
#pragma unroll
        for (int i = 0; i < KW; i += 4) {
          const float4 q4 = *reinterpret_cast<const float4*>(qg_s + l * DK + k0 + i);
          const float4 w4 = *reinterpret_cast<const float4*>(w_s + l * DK + k0 + i);
          a[i] = fmaf(q4.x, d, fmaf(w4.x, g, a[i]));
          a[i + 1] = fmaf(q4.y, d, fmaf(w4.y, g, a[i + 1]));
          a[i + 2] = fmaf(q4.z, d, fmaf(w4.z, g, a[i + 2]));
          a[i + 3] = fmaf(q4.w, d, fmaf(w4.w, g, a[i + 3]));
        }
      }
      __syncthreads();  // (4) and (5) on other warps have finished reading dS
#pragma unroll
      for (int i = 0; i < KW; ++i) ds_s[(k0 + i) * SP + lane] = a[i];
    }
    __syncthreads();
  }
}

template <int DK>
void launch_fwd(const float* W, const float* U, const float* QG, const float* M, const float* KD, const float* GL, float* O,
                float* Sstart, int BH, int C, int dv, cudaStream_t stream) {
  const size_t smem = (size_t)(3 * L * DK + L * L + L * DVB + L * VP + DK * SP) * sizeof(float);
  auto kern = gdn_scan_fwd_kernel<DK>;
  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    configured = true;
  }
  kern<<<dim3(BH, dv / DVB), kThreads, smem, stream>>>(W, U, QG, M, KD, GL, O, Sstart, C, dv);
}

template <int DK>
void launch_bwd(const float* W, const float* U, const float* QG, const float* M, const float* KD, const float* GL,
                const float* Sstart, const float* dO, float* dW, float* dU, float* dQG, float* dM, float* dKD, float* dGL,
                int BH, int C, int dv, cudaStream_t stream) {
  const size_t smem = (size_t)(3 * L * DK + L * L + L * DVB + 3 * L * VP + 2 * DK * SP) * sizeof(float);
  auto kern = gdn_scan_bwd_kernel<DK>;
  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    configured = true;
  }
  kern<<<dim3(BH, dv / DVB), kThreads, smem, stream>>>(W, U, QG, M, KD, GL, Sstart, dO, dW, dU, dQG, dM, dKD, dGL, C, dv);
}

}  // namespace

bool gdn_scan_supported(int dk, int dv) { return (dk == 64 || dk == 128) && dv % DVB == 0 && dv > 0; }

void gdn_scan_fwd(const float* W, const float* U, const float* QG, const float* M, const float* KD, const float* GL,
                  float* O, float* Sstart, int BH, int C, int dk, int dv, cudaStream_t stream) {
  if (!gdn_scan_supported(dk, dv)) throw std::runtime_error("gdn_scan: key dim must be 64 or 128 and value dim a multiple of 32");
  if (BH == 0 || C == 0) return;
  if (dk == 64) launch_fwd<64>(W, U, QG, M, KD, GL, O, Sstart, BH, C, dv, stream);
  else launch_fwd<128>(W, U, QG, M, KD, GL, O, Sstart, BH, C, dv, stream);
}

// dW, dQG, dKD, dM, dGL are accumulated into (zero them first); dU is written.
void gdn_scan_bwd(const float* W, const float* U, const float* QG, const float* M, const float* KD, const float* GL,
                  const float* Sstart, const float* dO, float* dW, float* dU, float* dQG, float* dM, float* dKD,
                  float* dGL, int BH, int C, int dk, int dv, cudaStream_t stream) {
  if (!gdn_scan_supported(dk, dv)) throw std::runtime_error("gdn_scan: key dim must be 64 or 128 and value dim a multiple of 32");
  if (BH == 0 || C == 0) return;
  if (dk == 64) launch_bwd<64>(W, U, QG, M, KD, GL, Sstart, dO, dW, dU, dQG, dM, dKD, dGL, BH, C, dv, stream);
  else launch_bwd<128>(W, U, QG, M, KD, GL, Sstart, dO, dW, dU, dQG, dM, dKD, dGL, BH, C, dv, stream);
}

}  // namespace mt
