// FP8 GEMM with per-tensor scales for sm_100a:  C[M,N] (bf16) = out_scale * A[M,K] * B[N,K]^T,
// A and B 8-bit floats (e4m3 or e5m2, chosen per operand), fp32 accumulation in tensor memory with
// tcgen05.mma.kind::f8f6f4 (K = 32 per instruction).  Both operands K-major; the quantise kernels below write the
// transposed copy where a layer needs one.  Same persistent warp-specialised structure as the bf16 GEMM: warp 0 TMA
// producer (128x128-byte A tiles, 256x128-byte B tiles, 4-stage ring), warp 1 MMA issuer, warps 2-5 epilogue with
// double-buffered accumulators; `out_scale` is read from device memory (1 / (scale_a * scale_b)), so no host
// synchronisation sits between the amax reduction and the GEMM.
//
// Per-tensor dynamic scaling follows the reference's fp8 recipe (mintext/modules/linear.py:37-57): activations to
// e4m3 with 448/amax, weights to e5m2 with 57344/amax.
#include "../common/ptx.cuh"
#include "../common/tmap.h"
#include "../common/pair.cuh"
#include "../api.h"
#include <cuda_fp8.h>
#include <cstdlib>

namespace mt {
namespace {

constexpr int BM = 128, BN = 256, BK = 128, UMMA_K = 32;  // BK bytes = one 128-byte swizzle span
constexpr int kEpiWarps = 4;
constexpr int kThreads = 32 * (2 + kEpiWarps);
constexpr int kEpiStageBytes = 4096;
constexpr int kStages = 4;

struct FCfg {
  static constexpr int A_BYTES = BM * BK, B_BYTES = BN * BK, STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int EPI_BYTES = kEpiWarps * 2 * kEpiStageBytes;
  static constexpr int OFF_EPI = kStages * STAGE_BYTES;
  static constexpr int OFF_BAR = OFF_EPI + EPI_BYTES;
  static constexpr int SMEM_BYTES = OFF_BAR + 256;
  static constexpr int TMEM_COLS = 2 * BN;
  static_assert(SMEM_BYTES <= 232448, "shared memory budget");
};

__device__ __forceinline__ void tile_coord(int tile, int num_m, int num_n, int& m_idx, int& n_idx) {
  const int per_group = 8 * num_m;
  const int group = tile / per_group;
  const int first_n = group * 8;
  const int gsize = min(8, num_n - first_n);
  const int local = tile - group * per_group;
  m_idx = local / gsize;
  n_idx = first_n + local % gsize;
}

__global__ void __launch_bounds__(kThreads, 1)
gemm_fp8_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                const __grid_constant__ CUtensorMap tmC, int M, int N, int K, int a_fmt, int b_fmt,
                const float* __restrict__ scale_a, const float* __restrict__ scale_b, int* status) {
  using C = FCfg;
  extern __shared__ __align__(1024) uint8_t smem[];
  if ((smem_u32(smem) & 1023u) != 0) {
    if (threadIdx.x == 0 && status) atomicCAS(status, 0, MT_ERR_BAD_ARGS);
    return;
  }
  uint8_t* epi_base = smem + C::OFF_EPI;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::OFF_BAR);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + kStages;
  uint64_t* tmem_full = bars + 2 * kStages;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_m = (M + BM - 1) / BM;
  const int num_n = (N + BN - 1) / BN;
  const int num_tiles = num_m * num_n;
  const int num_kb = (K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tmem_full[b], 1);
      mbar_init(&tmem_empty[b], kEpiWarps);
    }
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmB);
    prefetch_tmap(&tmC);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      int it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int m_idx, n_idx;
        tile_coord(tile, num_m, num_n, m_idx, n_idx);
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % kStages;
          if (!mbar_wait(&empty_bar[s], ((it / kStages) & 1) ^ 1, abort_flag, status, MT_ERR_TIMEOUT_EMPTY)) {
            ok = false;
            break;
          }
          uint8_t* a_dst = smem + s * C::STAGE_BYTES;
          mbar_expect_tx(&full_bar[s], C::STAGE_BYTES);
          tma_load_2d(a_dst, &tmA, &full_bar[s], kb * BK, m_idx * BM);
          tma_load_2d(a_dst + C::A_BYTES, &tmB, &full_bar[s], kb * BK, n_idx * BN);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = make_idesc_f8(BM, BN, a_fmt, b_fmt);
      int it = 0, tcount = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++tcount) {
        const int buf = tcount & 1;
        if (!mbar_wait(&tmem_empty[buf], ((tcount >> 1) & 1) ^ 1, abort_flag, status, MT_ERR_TIMEOUT_TMEM_EMPTY)) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + buf * BN;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % kStages;
          if (!mbar_wait(&full_bar[s], (it / kStages) & 1, abort_flag, status, MT_ERR_TIMEOUT_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(smem + s * C::STAGE_BYTES);
          const uint32_t b_addr = a_addr + C::A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            tc_mma_f8(d_tmem, make_smem_desc_sw128(a_addr + k * UMMA_K, 16, 1024),
                      make_smem_desc_sw128(b_addr + k * UMMA_K, 16, 1024), idesc, (kb | k) != 0 ? 1u : 0u);
          tc_commit(&empty_bar[s]);
        }
        if (ok) tc_commit(&tmem_full[buf]);
      }
    }
  } else {
    const int q = warp & 3;
    uint8_t* stage0 = epi_base + (warp - 2) * 2 * kEpiStageBytes;
    const float out_scale = 1.f / (scale_a[0] * scale_b[0]);
    int tcount = 0, nstores = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++tcount) {
      int m_idx, n_idx;
      tile_coord(tile, num_m, num_n, m_idx, n_idx);
      const int buf = tcount & 1;
      if (!mbar_wait_warp(&tmem_full[buf], (tcount >> 1) & 1, abort_flag, status, MT_ERR_TIMEOUT_TMEM_FULL)) break;
      tc_fence_after_sync();
      const int row0 = m_idx * BM + q * 32;
      const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * BN;
      for (int c = 0; c < BN / 64; ++c) {
        const int col0 = n_idx * BN + c * 64;
        if (col0 >= N) break;
        uint8_t* sbuf = stage0 + (nstores & 1) * kEpiStageBytes;
        if (lane == 0) tma_wait_group_read<1>();
        __syncwarp();
        uint8_t* srow = sbuf + lane * 128;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(t_lane + c * 64 + h * 32, r);
          tc_wait_ld();
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint4 v;
            v.x = pack_bf16x2(__uint_as_float(r[8 * j + 0]) * out_scale, __uint_as_float(r[8 * j + 1]) * out_scale);
            v.y = pack_bf16x2(__uint_as_float(r[8 * j + 2]) * out_scale, __uint_as_float(r[8 * j + 3]) * out_scale);
            v.z = pack_bf16x2(__uint_as_float(r[8 * j + 4]) * out_scale, __uint_as_float(r[8 * j + 5]) * out_scale);
            v.w = pack_bf16x2(__uint_as_float(r[8 * j + 6]) * out_scale, __uint_as_float(r[8 * j + 7]) * out_scale);
            *reinterpret_cast<uint4*>(srow + (((h * 4 + j) ^ (lane & 7)) << 4)) = v;
          }
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          if (row0 < M) tma_store_2d(&tmC, sbuf, col0, row0);
          tma_commit_group();
        }
        ++nstores;
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[buf]);
    }
    if (lane == 0) tma_wait_group<0>();
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    __syncwarp();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}


// ---------------------------------------------------------------------------------------- CTA-pair version
// Same product on a 2-CTA cluster (tcgen05 cta_group::2): 256x256 tile per pair, each CTA stages 128 rows of A and
// 128 rows of B (32 KB per stage, six stages); protocol as in dense_bf16_2cta.cu.
constexpr int kPairStages = 6;
struct FPCfg {
  static constexpr int A_BYTES = BM * BK, B_BYTES = (BN / 2) * BK, STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int EPI_BYTES = kEpiWarps * 2 * kEpiStageBytes;
  static constexpr int OFF_EPI = kPairStages * STAGE_BYTES;
  static constexpr int OFF_BAR = OFF_EPI + EPI_BYTES;
  static constexpr int SMEM_BYTES = OFF_BAR + 256;
  static constexpr int TMEM_COLS = 2 * BN;
  static_assert(SMEM_BYTES <= 232448, "shared memory budget");
};

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
gemm_fp8_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                     const __grid_constant__ CUtensorMap tmC, int M, int N, int K, int a_fmt, int b_fmt,
                     const float* __restrict__ scale_a, const float* __restrict__ scale_b, int* status) {
  using C = FPCfg;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* epi_base = smem + C::OFF_EPI;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::OFF_BAR);
  uint64_t* full_bar = bars;                        // leader only
  uint64_t* empty_bar = bars + kPairStages;         // per CTA
  uint64_t* tmem_full = bars + 2 * kPairStages;     // per CTA
  uint64_t* tmem_empty = tmem_full + 2;             // leader only (8 arrivals)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  const int num_m = (M + 2 * BM - 1) / (2 * BM);
  const int num_n = (N + BN - 1) / BN;
  const int num_tiles = num_m * num_n;
  const int num_kb = (K + BK - 1) / BK;
  const bool aligned = (smem_u32(smem) & 1023u) == 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kPairStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tmem_full[b], 1);
      mbar_init(&tmem_empty[b], 2 * kEpiWarps);
    }
    *abort_flag = aligned ? 0 : 1;
    if (!aligned && status) atomicCAS(status, 0, MT_ERR_BAD_ARGS);
    fence_barrier_init();
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmB);
    prefetch_tmap(&tmC);
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, C::TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0 && aligned) {
      int it = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        int m_idx, n_idx;
        tile_coord(tile, num_m, num_n, m_idx, n_idx);
        const int row0 = m_idx * (2 * BM) + rank * BM;
        const int col0 = n_idx * BN + rank * (BN / 2);
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % kPairStages;
          if (!mbar_wait(&empty_bar[s], ((it / kPairStages) & 1) ^ 1, abort_flag, status, MT_ERR_TIMEOUT_EMPTY)) {
            ok = false;
            break;
          }
          uint8_t* a_dst = smem + s * C::STAGE_BYTES;
          if (leader) mbar_expect_tx(&full_bar[s], 2 * C::STAGE_BYTES);
          tma_load_2d_pair(a_dst, &tmA, &full_bar[s], kb * BK, row0);
          tma_load_2d_pair(a_dst + C::A_BYTES, &tmB, &full_bar[s], kb * BK, col0);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && leader && aligned) {
      const uint32_t idesc = make_idesc_f8(2 * BM, BN, a_fmt, b_fmt);
      int it = 0, tcount = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, ++tcount) {
        const int buf = tcount & 1;
        if (!mbar_wait(&tmem_empty[buf], ((tcount >> 1) & 1) ^ 1, abort_flag, status, MT_ERR_TIMEOUT_TMEM_EMPTY)) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + buf * BN;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % kPairStages;
          if (!mbar_wait(&full_bar[s], (it / kPairStages) & 1, abort_flag, status, MT_ERR_TIMEOUT_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(smem + s * C::STAGE_BYTES);
          const uint32_t b_addr = a_addr + C::A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            tc_mma_f8_pair(d_tmem, make_smem_desc_sw128(a_addr + k * UMMA_K, 16, 1024),
                           make_smem_desc_sw128(b_addr + k * UMMA_K, 16, 1024), idesc, (kb | k) != 0 ? 1u : 0u);
          tc_commit_pair(&empty_bar[s]);
        }
        if (ok) tc_commit_pair(&tmem_full[buf]);
      }
    }
  } else {
    const int q = warp & 3;
    uint8_t* stage0 = epi_base + (warp - 2) * 2 * kEpiStageBytes;
    const float out_scale = 1.f / (scale_a[0] * scale_b[0]);
    int tcount = 0, nstores = 0;
    for (int tile = pair; tile < num_tiles && aligned; tile += num_pairs, ++tcount) {
      int m_idx, n_idx;
      tile_coord(tile, num_m, num_n, m_idx, n_idx);
      const int buf = tcount & 1;
      if (!mbar_wait_warp(&tmem_full[buf], (tcount >> 1) & 1, abort_flag, status, MT_ERR_TIMEOUT_TMEM_FULL)) break;
      tc_fence_after_sync();
      const int row0 = m_idx * (2 * BM) + rank * BM + q * 32;
      const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * BN;
      for (int c = 0; c < BN / 64; ++c) {
        const int col0 = n_idx * BN + c * 64;
        if (col0 >= N) break;
        uint8_t* sbuf = stage0 + (nstores & 1) * kEpiStageBytes;
        if (lane == 0) tma_wait_group_read<1>();
        __syncwarp();
        uint8_t* srow = sbuf + lane * 128;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(t_lane + c * 64 + h * 32, r);
          tc_wait_ld();
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint4 v;
            v.x = pack_bf16x2(__uint_as_float(r[8 * j + 0]) * out_scale, __uint_as_float(r[8 * j + 1]) * out_scale);
            v.y = pack_bf16x2(__uint_as_float(r[8 * j + 2]) * out_scale, __uint_as_float(r[8 * j + 3]) * out_scale);
            v.z = pack_bf16x2(__uint_as_float(r[8 * j + 4]) * out_scale, __uint_as_float(r[8 * j + 5]) * out_scale);
            v.w = pack_bf16x2(__uint_as_float(r[8 * j + 6]) * out_scale, __uint_as_float(r[8 * j + 7]) * out_scale);
            *reinterpret_cast<uint4*>(srow + (((h * 4 + j) ^ (lane & 7)) << 4)) = v;
          }
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          if (row0 < M) tma_store_2d(&tmC, sbuf, col0, row0);
          tma_commit_group();
        }
        ++nstores;
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_leader(&tmem_empty[buf]);
    }
    if (lane == 0) tma_wait_group<0>();
  }

  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after_sync();
    __syncwarp();
    tmem_dealloc_pair(tmem_base, C::TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------------- quantisation
__global__ void amax_kernel(const __nv_bfloat16* __restrict__ x, int64_t n, float* __restrict__ amax) {
  float m = 0.f;
  const int64_t nvec = n >> 3;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (int64_t)gridDim.x * blockDim.x) {
    const uint4 v = reinterpret_cast<const uint4*>(x)[i];
    const __nv_bfloat16* h = reinterpret_cast<const __nv_bfloat16*>(&v);
#pragma unroll
    for (int j = 0; j < 8; ++j) m = fmaxf(m, fabsf(__bfloat162float(h[j])));
  }
  for (int64_t i = (nvec << 3) + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x)
    m = fmaxf(m, fabsf(__bfloat162float(x[i])));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if ((threadIdx.x & 31) == 0) atomicMax(reinterpret_cast<int*>(amax), __float_as_int(m));  // m >= 0: int order = float order
}

template <bool E5M2>
__device__ __forceinline__ uint8_t to_fp8(float v) {
  return static_cast<uint8_t>(__nv_cvt_float_to_fp8(v, __NV_SATFINITE, E5M2 ? __NV_E5M2 : __NV_E4M3));
}

// scale[0] = fmax / max(amax, 1e-12); q = fp8(x * scale); optionally also the transposed copy qt[C, R].
template <bool E5M2>
__global__ void quantize_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ amax,
                                float* __restrict__ scale, uint8_t* __restrict__ q, uint8_t* __restrict__ qt, int R, int C) {
  __shared__ uint8_t tile[64][65];
  const float sc = (E5M2 ? 57344.f : 448.f) / fmaxf(amax[0], 1e-12f);
  if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) scale[0] = sc;
  const int r0 = blockIdx.y * 64, c0 = blockIdx.x * 64;
  const int tx = threadIdx.x & 63, ty = threadIdx.x >> 6;  // 256 threads: 64 columns x 4 row phases
  for (int rr = ty; rr < 64; rr += 4) {
    const int r = r0 + rr, c = c0 + tx;
    uint8_t v = 0;
    if (r < R && c < C) {
      v = to_fp8<E5M2>(__bfloat162float(x[(int64_t)r * C + c]) * sc);
      if (q) q[(int64_t)r * C + c] = v;
    }
    tile[rr][tx] = v;
  }
  if (qt == nullptr) return;
  __syncthreads();
  for (int cc = ty; cc < 64; cc += 4) {
    const int c = c0 + cc, r = r0 + tx;
    if (r < R && c < C) qt[(int64_t)c * R + r] = tile[tx][cc];
  }
}

// Flat variant (no transposed copy): 16 elements per thread, 32 bytes in, 16 bytes out.
template <bool E5M2>
__global__ void quantize_flat_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ amax,
                                     float* __restrict__ scale, uint8_t* __restrict__ q, int64_t n16) {
  const float sc = (E5M2 ? 57344.f : 448.f) / fmaxf(amax[0], 1e-12f);
  if (blockIdx.x == 0 && threadIdx.x == 0) scale[0] = sc;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += (int64_t)gridDim.x * blockDim.x) {
    const uint4 a = reinterpret_cast<const uint4*>(x)[2 * i];
    const uint4 b = reinterpret_cast<const uint4*>(x)[2 * i + 1];
    const __nv_bfloat16* ha = reinterpret_cast<const __nv_bfloat16*>(&a);
    const __nv_bfloat16* hb = reinterpret_cast<const __nv_bfloat16*>(&b);
    union {
      uint4 u;
      uint8_t c[16];
    } o;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      o.c[j] = to_fp8<E5M2>(__bfloat162float(ha[j]) * sc);
      o.c[8 + j] = to_fp8<E5M2>(__bfloat162float(hb[j]) * sc);
    }
    reinterpret_cast<uint4*>(q)[i] = o.u;
  }
}

}  // namespace

void fp8_amax(const void* x, int64_t n, float* amax, cudaStream_t stream) {
  cudaMemsetAsync(amax, 0, sizeof(float), stream);
  if (n == 0) return;
  int64_t blocks = (n / 8 + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  if (blocks < 1) blocks = 1;
  amax_kernel<<<(int)blocks, 256, 0, stream>>>((const __nv_bfloat16*)x, n, amax);
}

void fp8_quantize(const void* x, const float* amax, float* scale, void* q, void* qt, int R, int C, bool e5m2,
                  cudaStream_t stream) {
  if (R == 0 || C == 0) return;
  const int64_t n = (int64_t)R * C;
  if (qt == nullptr && n % 16 == 0) {
    int64_t blocks = (n / 16 + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (e5m2) quantize_flat_kernel<true><<<(int)blocks, 256, 0, stream>>>((const __nv_bfloat16*)x, amax, scale, (uint8_t*)q, n / 16);
    else quantize_flat_kernel<false><<<(int)blocks, 256, 0, stream>>>((const __nv_bfloat16*)x, amax, scale, (uint8_t*)q, n / 16);
    return;
  }
  dim3 grid((C + 63) / 64, (R + 63) / 64);
  if (e5m2)
    quantize_kernel<true><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)x, amax, scale, (uint8_t*)q, (uint8_t*)qt, R, C);
  else
    quantize_kernel<false><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)x, amax, scale, (uint8_t*)q, (uint8_t*)qt, R, C);
}

void gemm_fp8(const void* A, const void* B, void* Cout, int M, int N, int K, bool a_e5m2, bool b_e5m2,
              const float* scale_a, const float* scale_b, int* status, int num_sms, cudaStream_t stream) {
  if (K % 16 != 0 || N % 8 != 0) throw std::runtime_error("gemm_fp8: K must be a multiple of 16 and N of 8");
  const auto u8 = CU_TENSOR_MAP_DATA_TYPE_UINT8;
  const auto sw = CU_TENSOR_MAP_SWIZZLE_128B;
  CUtensorMap tA = make_tmap_2d(A, u8, 1, M, K, K, BM, BK, sw);
  CUtensorMap tC = make_tmap_2d(Cout, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, N, N, 32, 64, sw);
  static const bool single_only = [] {
    const char* e = std::getenv("MT_GEMM_SINGLE_CTA");
    return e != nullptr && e[0] == '1';
  }();
  if (!single_only && M > 128 && N > 128) {  // CTA pairs: each CTA loads half of the B tile
    CUtensorMap tBh = make_tmap_2d(B, u8, 1, N, K, K, BN / 2, BK, sw);
    static bool pair_configured = false;
    if (!pair_configured) {
      MT_CUDA_CHECK(cudaFuncSetAttribute(gemm_fp8_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FPCfg::SMEM_BYTES));
      pair_configured = true;
    }
    const int ptiles = ((M + 2 * BM - 1) / (2 * BM)) * ((N + BN - 1) / BN);
    const int pairs = ptiles < num_sms / 2 ? ptiles : num_sms / 2;
    gemm_fp8_pair_kernel<<<2 * pairs, kThreads, FPCfg::SMEM_BYTES, stream>>>(tA, tBh, tC, M, N, K, a_e5m2 ? 1 : 0,
                                                                            b_e5m2 ? 1 : 0, scale_a, scale_b, status);
    MT_CUDA_CHECK(cudaGetLastError());
    return;
  }
  CUtensorMap tB = make_tmap_2d(B, u8, 1, N, K, K, BN, BK, sw);
  static bool configured = false;
  if (!configured) {
    MT_CUDA_CHECK(cudaFuncSetAttribute(gemm_fp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FCfg::SMEM_BYTES));
    configured = true;
  }
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  const int grid = tiles < num_sms ? tiles : num_sms;
  if (grid == 0) return;
  gemm_fp8_kernel<<<grid, kThreads, FCfg::SMEM_BYTES, stream>>>(tA, tB, tC, M, N, K, a_e5m2 ? 1 : 0, b_e5m2 ? 1 : 0,
                                                                 scale_a, scale_b, status);
  MT_CUDA_CHECK(cudaGetLastError());
}

}  // namespace mt
