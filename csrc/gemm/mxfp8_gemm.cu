// MXFP8 GEMM for sm_100a:  C[M,N] (bf16) = A[M,K] * B[N,K]^T with block-scaled 8-bit operands: e4m3 elements and one
// power-of-two scale (UE8M0 byte) per 32 consecutive elements along K, applied by the tensor core itself
// (tcgen05.mma.kind::mxf8f6f4.block_scale, K = 32 per instruction, fp32 accumulation in tensor memory).
//
// Scale factors reach the MMA through tensor memory.  For an operand tile of up to 128 rows and one 128-element
// k-block the hardware wants, on lane (row % 32), the 32-bit column (row / 32) holding the four scale bytes of the
// k-block's four 32-element groups; the instruction descriptor's scale-id fields pick the byte.  The quantise kernel
// therefore writes the scales of every (row tile, k-block) as "atoms" of 512 bytes = 32 lanes x 16 bytes
// (byte (row%32)*16 + (row%128/32)*4 + group), tile-relative, one atom per 128 rows of the tile: a 128-row A tile
// has one atom per k-block, a 192-row B tile two.  The producer brings the atoms of a k-block into shared memory
// with one bulk copy per operand next to the TMA tile loads, and the MMA thread moves them into tensor memory with
// tcgen05.cp (32x128b.warpx4: every 32-lane quarter receives the same 32 x 16 bytes) right before the four MMAs of
// the k-block; two alternating column sets keep the copies of the next k-block off the scales still in use.
//
// Structure as in the per-tensor FP8 kernel: persistent CTAs, warp 0 TMA producer (4-stage ring), warp 1 MMA
// issuer, warps 2-5 epilogue; tiles are 128 x 192 so that two accumulators (384 columns) and the scale columns fit
// the 512 columns of tensor memory and the epilogue of one tile overlaps the main loop of the next.
//
// The scale of a block is the smallest power of two that brings the block's largest magnitude within the e4m3
// range (448); quantisation needs no tensor-wide amax pass.  Layer semantics (which products run in 8 bits) follow
// mintext/modules/linear.py:37-57.
#include "../common/ptx.cuh"
#include "../common/tmap.h"
#include "../api.h"
#include <cuda_fp8.h>

namespace mt {
namespace {

constexpr int BM = 128, BN = 192, BK = 128, UMMA_K = 32;  // BK bytes = one 128-byte swizzle span
constexpr int kEpiWarps = 4;
constexpr int kThreads = 32 * (2 + kEpiWarps);
constexpr int kEpiStageBytes = 4096;
constexpr int kStages = 4;
constexpr int kAtomBytes = 512;

struct XCfg {
  static constexpr int A_BYTES = BM * BK, B_BYTES = BN * BK, STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int SFA_BYTES = kAtomBytes, SFB_BYTES = 2 * kAtomBytes, SF_STAGE_BYTES = SFA_BYTES + SFB_BYTES;
  static constexpr int OFF_SF = kStages * STAGE_BYTES;
  static constexpr int OFF_EPI = OFF_SF + kStages * SF_STAGE_BYTES;
  static constexpr int EPI_BYTES = kEpiWarps * 2 * kEpiStageBytes;
  static constexpr int OFF_BAR = OFF_EPI + EPI_BYTES;
  static constexpr int SMEM_BYTES = OFF_BAR + 256;
  static constexpr int TMEM_COLS = 512;
  static constexpr int COL_SFA = 2 * BN, COL_SFB = COL_SFA + 8;  // two sets each: 4 columns for A, 8 for B
  static_assert(STAGE_BYTES % 1024 == 0 && OFF_EPI % 1024 == 0, "swizzled tiles need 1024-byte alignment");
  static_assert(COL_SFB + 16 <= TMEM_COLS, "tensor memory budget");
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

// Shared-memory descriptor without swizzling: 8-row x 16-byte core matrices, `sbo_bytes` apart along the rows.
__device__ __forceinline__ uint64_t make_smem_desc_plain(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= static_cast<uint64_t>(1) << 46;  // descriptor version (Blackwell)
  return d;
}

// 32 rows x 16 bytes of shared memory -> 4 columns of tensor memory, replicated into all four lane quarters.
__device__ __forceinline__ void tc_cp_32x128b_warpx4(uint32_t tmem_dst, uint64_t desc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(tmem_dst), "l"(desc) : "memory");
}

__device__ __forceinline__ void tc_mma_mxf8(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                            uint32_t tmem_sfa, uint32_t tmem_sfb, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(tmem_sfa), "r"(tmem_sfb)
      : "memory");
}

// Block-scaled instruction descriptor: e4m3 x e4m3 (format 0), K-major operands, UE8M0 scales, scale byte `sf_id`
// of the 32-bit scale column for both operands.
__host__ __device__ constexpr uint32_t make_idesc_mxf8(int M, int N, uint32_t sf_id) {
  return (sf_id << 4) | (static_cast<uint32_t>(N >> 3) << 17) | (1u << 23) | (static_cast<uint32_t>(M >> 4) << 24) |
         (sf_id << 29);
}

__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(smem_dst)),
               "l"(reinterpret_cast<uint64_t>(gsrc)), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

__global__ void __launch_bounds__(kThreads, 1)
gemm_mxfp8_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                  const __grid_constant__ CUtensorMap tmC, const uint8_t* __restrict__ sfa,
                  const uint8_t* __restrict__ sfb, int M, int N, int K, int* status) {
  using C = XCfg;
  extern __shared__ __align__(1024) uint8_t smem[];
  if ((smem_u32(smem) & 1023u) != 0) {
    if (threadIdx.x == 0 && status) atomicCAS(status, 0, MT_ERR_BAD_ARGS);
    return;
  }
  uint8_t* sf_base = smem + C::OFF_SF;
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
  const int num_kb = K / BK;

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
        const uint8_t* sfa_row = sfa + static_cast<int64_t>(m_idx) * num_kb * C::SFA_BYTES;
        const uint8_t* sfb_row = sfb + static_cast<int64_t>(n_idx) * num_kb * C::SFB_BYTES;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % kStages;
          if (!mbar_wait(&empty_bar[s], ((it / kStages) & 1) ^ 1, abort_flag, status, MT_ERR_TIMEOUT_EMPTY)) {
            ok = false;
            break;
          }
          uint8_t* a_dst = smem + s * C::STAGE_BYTES;
          uint8_t* sf_dst = sf_base + s * C::SF_STAGE_BYTES;
          mbar_expect_tx(&full_bar[s], C::STAGE_BYTES + C::SF_STAGE_BYTES);
          tma_load_2d(a_dst, &tmA, &full_bar[s], kb * BK, m_idx * BM);
          tma_load_2d(a_dst + C::A_BYTES, &tmB, &full_bar[s], kb * BK, n_idx * BN);
          bulk_g2s(sf_dst, sfa_row + kb * C::SFA_BYTES, C::SFA_BYTES, &full_bar[s]);
          bulk_g2s(sf_dst + C::SFA_BYTES, sfb_row + kb * C::SFB_BYTES, C::SFB_BYTES, &full_bar[s]);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
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
          const uint32_t sf_addr = smem_u32(sf_base + s * C::SF_STAGE_BYTES);
          const uint32_t t_sfa = tmem_base + C::COL_SFA + (it & 1) * 4;
          const uint32_t t_sfb = tmem_base + C::COL_SFB + (it & 1) * 8;
          tc_cp_32x128b_warpx4(t_sfa, make_smem_desc_plain(sf_addr, 16, 128));
          tc_cp_32x128b_warpx4(t_sfb, make_smem_desc_plain(sf_addr + C::SFA_BYTES, 16, 128));
          tc_cp_32x128b_warpx4(t_sfb + 4, make_smem_desc_plain(sf_addr + C::SFA_BYTES + kAtomBytes, 16, 128));
          const uint64_t da = make_smem_desc_sw128(a_addr, 16, 1024), db = make_smem_desc_sw128(b_addr, 16, 1024);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            tc_mma_mxf8(d_tmem, da + k * (UMMA_K >> 4), db + k * (UMMA_K >> 4), make_idesc_mxf8(BM, BN, k), t_sfa, t_sfb,
                        (kb | k) != 0 ? 1u : 0u);
          tc_commit(&empty_bar[s]);
        }
        if (ok) tc_commit(&tmem_full[buf]);
      }
    }
  } else {
    const int q = warp & 3;
    uint8_t* stage0 = epi_base + (warp - 2) * 2 * kEpiStageBytes;
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
            v.x = pack_bf16x2(__uint_as_float(r[8 * j + 0]), __uint_as_float(r[8 * j + 1]));
            v.y = pack_bf16x2(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3]));
            v.z = pack_bf16x2(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5]));
            v.w = pack_bf16x2(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7]));
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


// ---------------------------------------------------------------------------------------- grouped (expert) product
// Y[rows, N] = X[rows, K] * W[e]^T-view for the rows of expert e, block-scaled like the dense kernel above.  Rows are
// grouped by expert at 128-aligned offsets (`offsets`, device int32[E+1]), so every 128-row A tile belongs to one
// expert and its scale atoms are indexed by the global row block exactly as in the dense case.  The B operand is the
// stack of per-expert matrices [E, N, K] (K-major, e4m3) with per-expert scale tiling (192-row tiles inside each
// expert; rows beyond N are zero-filled by the 3-D tile load, never the next expert's).  Tiles are (row block,
// 192-column block); the expert of a row block comes from a table built in shared memory at kernel start.
constexpr int kMaxRowBlocks = 4096;

__global__ void __launch_bounds__(kThreads, 1)
grouped_mxfp8_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                     const __grid_constant__ CUtensorMap tmC, const uint8_t* __restrict__ sfa,
                     const uint8_t* __restrict__ sfb, const int* __restrict__ offsets, int E, int N, int K, int* status) {
  using C = XCfg;
  extern __shared__ __align__(1024) uint8_t smem[];
  if ((smem_u32(smem) & 1023u) != 0) {
    if (threadIdx.x == 0 && status) atomicCAS(status, 0, MT_ERR_BAD_ARGS);
    return;
  }
  uint8_t* sf_base = smem + C::OFF_SF;
  uint8_t* epi_base = smem + C::OFF_EPI;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::OFF_BAR);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + kStages;
  uint64_t* tmem_full = bars + 2 * kStages;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  uint16_t* mb2e = reinterpret_cast<uint16_t*>(smem + C::SMEM_BYTES);  // expert of every 128-row block

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_n = (N + BN - 1) / BN;
  const int num_kb = K / BK;
  int total_rows = offsets[E];
  if (total_rows > kMaxRowBlocks * BM) total_rows = kMaxRowBlocks * BM;
  const int num_mb = total_rows / BM;
  const int num_tiles = num_mb * num_n;
  for (int e = 0; e < E; ++e) {  // every thread fills its share of each expert's row blocks
    const int b0 = offsets[e] / BM, b1 = min(offsets[e + 1] / BM, num_mb);
    for (int mb = b0 + (int)threadIdx.x; mb < b1; mb += blockDim.x) mb2e[mb] = (uint16_t)e;
  }

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
        const int mb = tile / num_n, n_idx = tile % num_n;
        const int e = mb2e[mb];
        const uint8_t* sfa_row = sfa + static_cast<int64_t>(mb) * num_kb * C::SFA_BYTES;
        const uint8_t* sfb_row = sfb + (static_cast<int64_t>(e) * num_n + n_idx) * num_kb * C::SFB_BYTES;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % kStages;
          if (!mbar_wait(&empty_bar[s], ((it / kStages) & 1) ^ 1, abort_flag, status, MT_ERR_TIMEOUT_EMPTY)) {
            ok = false;
            break;
          }
          uint8_t* a_dst = smem + s * C::STAGE_BYTES;
          uint8_t* sf_dst = sf_base + s * C::SF_STAGE_BYTES;
          mbar_expect_tx(&full_bar[s], C::STAGE_BYTES + C::SF_STAGE_BYTES);
          tma_load_2d(a_dst, &tmA, &full_bar[s], kb * BK, mb * BM);
          tma_load_3d(a_dst + C::A_BYTES, &tmB, &full_bar[s], kb * BK, n_idx * BN, e);
          bulk_g2s(sf_dst, sfa_row + kb * C::SFA_BYTES, C::SFA_BYTES, &full_bar[s]);
          bulk_g2s(sf_dst + C::SFA_BYTES, sfb_row + kb * C::SFB_BYTES, C::SFB_BYTES, &full_bar[s]);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
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
          const uint32_t sf_addr = smem_u32(sf_base + s * C::SF_STAGE_BYTES);
          const uint32_t t_sfa = tmem_base + C::COL_SFA + (it & 1) * 4;
          const uint32_t t_sfb = tmem_base + C::COL_SFB + (it & 1) * 8;
          tc_cp_32x128b_warpx4(t_sfa, make_smem_desc_plain(sf_addr, 16, 128));
          tc_cp_32x128b_warpx4(t_sfb, make_smem_desc_plain(sf_addr + C::SFA_BYTES, 16, 128));
          tc_cp_32x128b_warpx4(t_sfb + 4, make_smem_desc_plain(sf_addr + C::SFA_BYTES + kAtomBytes, 16, 128));
          const uint64_t da = make_smem_desc_sw128(a_addr, 16, 1024), db = make_smem_desc_sw128(b_addr, 16, 1024);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            tc_mma_mxf8(d_tmem, da + k * (UMMA_K >> 4), db + k * (UMMA_K >> 4), make_idesc_mxf8(BM, BN, k), t_sfa, t_sfb,
                        (kb | k) != 0 ? 1u : 0u);
          tc_commit(&empty_bar[s]);
        }
        if (ok) tc_commit(&tmem_full[buf]);
      }
    }
  } else {
    const int q = warp & 3;
    uint8_t* stage0 = epi_base + (warp - 2) * 2 * kEpiStageBytes;
    int tcount = 0, nstores = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++tcount) {
      const int mb = tile / num_n, n_idx = tile % num_n;
      const int buf = tcount & 1;
      if (!mbar_wait_warp(&tmem_full[buf], (tcount >> 1) & 1, abort_flag, status, MT_ERR_TIMEOUT_TMEM_FULL)) break;
      tc_fence_after_sync();
      const int row0 = mb * BM + q * 32;
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
            v.x = pack_bf16x2(__uint_as_float(r[8 * j + 0]), __uint_as_float(r[8 * j + 1]));
            v.y = pack_bf16x2(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3]));
            v.z = pack_bf16x2(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5]));
            v.w = pack_bf16x2(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7]));
            *reinterpret_cast<uint4*>(srow + (((h * 4 + j) ^ (lane & 7)) << 4)) = v;
          }
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          tma_store_2d(&tmC, sbuf, col0, row0);
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

// ---------------------------------------------------------------------------------------- quantisation
// Byte offset of the scale of (row, 32-element group `g32`) in a scale buffer whose row tiles are `T` rows
// (`atoms` = ceil(T / 128) atoms per tile and k-block), for a contraction length of `kb128` 128-element k-blocks.
__host__ __device__ __forceinline__ int64_t sf_offset(int row, int g32, int kb128, int T, int atoms) {
  const int tile = row / T, rr = row % T;
  return ((static_cast<int64_t>(tile) * kb128 + (g32 >> 2)) * atoms + (rr >> 7)) * kAtomBytes + (rr & 31) * 16 +
         ((rr & 127) >> 5) * 4 + (g32 & 3);
}

// Smallest e with amax * 2^-e <= 448, clamped to the UE8M0 range; an all-zero block gets the smallest scale.
__device__ __forceinline__ int mx_exponent(float amax) {
  const float t = amax * (1.f / 448.f);
  const int bits = __float_as_int(t);
  int e = ((bits >> 23) & 0xFF) - 127;
  if (bits & 0x7FFFFF) e += 1;
  return max(-127, min(e, 127));
}

__device__ __forceinline__ uint4 quantise16(const float (&v)[16], float inv) {
  union {
    uint4 u;
    uint8_t c[16];
  } o;
#pragma unroll
  for (int i = 0; i < 16; ++i)
    o.c[i] = static_cast<uint8_t>(__nv_cvt_float_to_fp8(v[i] * inv, __NV_SATFINITE, __NV_E4M3));
  return o.u;
}

// x [R, C] bf16 -> q [R, C] e4m3 with scales over 32-element groups along C (tile rows T), and / or the transposed
// copy qt [C, R] with scales over 32-element groups along R (tile rows Tt).  One 64 x 64 tile per block.
// blockIdx.z selects one matrix of a stack of `gridDim.z` equally shaped matrices (per-expert weights): element
// buffers advance by R*C per matrix, scale buffers by `sf_stride` / `sft_stride` bytes (each matrix has its own
// scale tiling, so a scale tile never spans two experts).
__global__ void mx_quantize_kernel(const __nv_bfloat16* __restrict__ x, int R, int C, uint8_t* __restrict__ q,
                                   uint8_t* __restrict__ sf, int T, uint8_t* __restrict__ qt, uint8_t* __restrict__ sft,
                                   int Tt, int64_t sf_stride, int64_t sft_stride) {
  __shared__ float tile[64][65];
  {
    const int64_t z = blockIdx.z, elems = static_cast<int64_t>(R) * C;
    x += z * elems;
    if (q != nullptr) { q += z * elems; sf += z * sf_stride; }
    if (qt != nullptr) { qt += z * elems; sft += z * sft_stride; }
  }
  const int r0 = blockIdx.y * 64, c0 = blockIdx.x * 64;
  const int sub = threadIdx.x >> 2, seg = threadIdx.x & 3;  // 64 rows (columns) x four 16-element segments
  {
    const int r = r0 + sub, c = c0 + seg * 16;
    float v[16];
    if (r < R && c < C) {  // C % 16 == 0: a segment is inside or outside as a whole
      const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<int64_t>(r) * C + c);
      const uint4 a = src[0], b = src[1];
      const __nv_bfloat16* ha = reinterpret_cast<const __nv_bfloat16*>(&a);
      const __nv_bfloat16* hb = reinterpret_cast<const __nv_bfloat16*>(&b);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        v[i] = __bfloat162float(ha[i]);
        v[8 + i] = __bfloat162float(hb[i]);
      }
    } else {
#pragma unroll
      for (int i = 0; i < 16; ++i) v[i] = 0.f;
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) tile[sub][seg * 16 + i] = v[i];
    if (q != nullptr) {
      float m = 0.f;
#pragma unroll
      for (int i = 0; i < 16; ++i) m = fmaxf(m, fabsf(v[i]));
      m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));  // the neighbouring segment completes the 32-element group
      const int e = mx_exponent(m);
      const float inv = __int_as_float((127 - e) << 23);
      if (r < R && c < C) {
        *reinterpret_cast<uint4*>(q + static_cast<int64_t>(r) * C + c) = quantise16(v, inv);
        if ((seg & 1) == 0) sf[sf_offset(r, c >> 5, C >> 7, T, (T + 127) >> 7)] = static_cast<uint8_t>(e + 127);
      }
    }
  }
  if (qt == nullptr) return;
  __syncthreads();
  {
    const int c = c0 + sub, r = r0 + seg * 16;  // this thread: column c, rows r .. r+15
    float v[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = tile[seg * 16 + i][sub];
    float m = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) m = fmaxf(m, fabsf(v[i]));
    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
    const int e = mx_exponent(m);
    const float inv = __int_as_float((127 - e) << 23);
    if (c < C && r < R) {  // R % 16 == 0
      *reinterpret_cast<uint4*>(qt + static_cast<int64_t>(c) * R + r) = quantise16(v, inv);
      if ((seg & 1) == 0) sft[sf_offset(c, r >> 5, R >> 7, Tt, (Tt + 127) >> 7)] = static_cast<uint8_t>(e + 127);
    }
  }
}

}  // namespace

int64_t mxfp8_sf_bytes(int rows, int K, bool b_operand) {
  const int T = b_operand ? BN : BM;
  const int64_t tiles = (rows + T - 1) / T;
  return tiles * (K / BK) * ((T + 127) / 128) * kAtomBytes;
}

// q / sf: element and scale buffers for groups along C; qt / sft: the same for the transposed copy (groups along
// R).  `*_b_operand` selects the scale tiling of the GEMM's B operand (192-row tiles) instead of A's (128-row tiles).
// Scale buffers hold mxfp8_sf_bytes(...) bytes and should be zero-filled once (padding rows are never written).
void mxfp8_quantize(const void* x, int R, int C, void* q, void* sf, bool q_b_operand, void* qt, void* sft,
                    bool qt_b_operand, cudaStream_t stream) {
  if (R == 0 || C == 0) return;
  if (C % 16 != 0) throw std::runtime_error("mxfp8_quantize: columns must be a multiple of 16");
  if (q != nullptr && C % BK != 0) throw std::runtime_error("mxfp8_quantize: row-wise groups need columns % 128 == 0");
  if (qt != nullptr && R % BK != 0) throw std::runtime_error("mxfp8_quantize: transposed groups need rows % 128 == 0");
  dim3 grid((C + 63) / 64, (R + 63) / 64);
  mx_quantize_kernel<<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(x), R, C, static_cast<uint8_t*>(q),
                                               static_cast<uint8_t*>(sf), q_b_operand ? BN : BM,
                                               static_cast<uint8_t*>(qt), static_cast<uint8_t*>(sft),
                                               qt_b_operand ? BN : BM, 0, 0);
  MT_CUDA_CHECK(cudaGetLastError());
}

// The same for a stack w [E, R, C] (expert weights), every matrix with its own B-operand scale tiling:
// q [E, R, C] with groups along C and scales sf (E * mxfp8_sf_bytes(R, C, true) bytes), and / or qt [E, C, R] with
// groups along R and scales sft (E * mxfp8_sf_bytes(C, R, true) bytes).
void mxfp8_quantize_stack(const void* w, int E, int R, int C, void* q, void* sf, void* qt, void* sft,
                          cudaStream_t stream) {
  if (E == 0 || R == 0 || C == 0) return;
  if (C % 16 != 0) throw std::runtime_error("mxfp8_quantize_stack: columns must be a multiple of 16");
  if (q != nullptr && C % BK != 0) throw std::runtime_error("mxfp8_quantize_stack: row-wise groups need columns % 128 == 0");
  if (qt != nullptr && R % BK != 0) throw std::runtime_error("mxfp8_quantize_stack: transposed groups need rows % 128 == 0");
  dim3 grid((C + 63) / 64, (R + 63) / 64, E);
  mx_quantize_kernel<<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(w), R, C, static_cast<uint8_t*>(q),
                                               static_cast<uint8_t*>(sf), BN, static_cast<uint8_t*>(qt),
                                               static_cast<uint8_t*>(sft), BN, mxfp8_sf_bytes(R, C, true),
                                               mxfp8_sf_bytes(C, R, true));
  MT_CUDA_CHECK(cudaGetLastError());
}

// Y [M_cap, N] bf16 = X [M_cap, K] (e4m3 + scales sfa, 128-row tiles) times, per expert, B[e] [N, K] (e4m3 + per-expert
// scales sfb); rows grouped by expert at the 128-aligned `offsets` (device int32[E+1]).
void grouped_gemm_mxfp8(const void* X, const void* sfa, const void* B, const void* sfb, void* Y, const int* offsets, int E,
                        int M_cap, int N, int K, int* status, int num_sms, cudaStream_t stream) {
  if (M_cap <= 0 || E <= 0) return;
  if (K % BK != 0 || N % 8 != 0) throw std::runtime_error("grouped_gemm_mxfp8: K must be a multiple of 128 and N of 8");
  if (M_cap % BM != 0 || M_cap / BM > kMaxRowBlocks || E > 65535)
    throw std::runtime_error("grouped_gemm_mxfp8: row capacity must be a multiple of 128 and at most 524288 rows");
  const auto u8 = CU_TENSOR_MAP_DATA_TYPE_UINT8;
  const auto sw = CU_TENSOR_MAP_SWIZZLE_128B;
  CUtensorMap tA = make_tmap_2d(X, u8, 1, M_cap, K, K, BM, BK, sw);
  CUtensorMap tB = make_tmap_3d(B, u8, 1, E, N, K, (uint64_t)N * K, K, 1, BN, BK, sw);
  CUtensorMap tC = make_tmap_2d(Y, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M_cap, N, N, 32, 64, sw);
  const int smem_bytes = XCfg::SMEM_BYTES + kMaxRowBlocks * (int)sizeof(uint16_t);
  static bool configured = false;
  if (!configured) {
    MT_CUDA_CHECK(cudaFuncSetAttribute(grouped_mxfp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
    configured = true;
  }
  grouped_mxfp8_kernel<<<num_sms, kThreads, smem_bytes, stream>>>(tA, tB, tC, static_cast<const uint8_t*>(sfa),
                                                                  static_cast<const uint8_t*>(sfb), offsets, E, N, K,
                                                                  status);
  MT_CUDA_CHECK(cudaGetLastError());
}

void gemm_mxfp8(const void* A, const void* sfa, const void* B, const void* sfb, void* Cout, int M, int N, int K,
                int* status, int num_sms, cudaStream_t stream) {
  if (K % BK != 0 || N % 8 != 0) throw std::runtime_error("gemm_mxfp8: K must be a multiple of 128 and N of 8");
  const auto u8 = CU_TENSOR_MAP_DATA_TYPE_UINT8;
  const auto sw = CU_TENSOR_MAP_SWIZZLE_128B;
  CUtensorMap tA = make_tmap_2d(A, u8, 1, M, K, K, BM, BK, sw);
  CUtensorMap tB = make_tmap_2d(B, u8, 1, N, K, K, BN, BK, sw);
  CUtensorMap tC = make_tmap_2d(Cout, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, N, N, 32, 64, sw);
  static bool configured = false;
  if (!configured) {
    MT_CUDA_CHECK(cudaFuncSetAttribute(gemm_mxfp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, XCfg::SMEM_BYTES));
    configured = true;
  }
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  const int grid = tiles < num_sms ? tiles : num_sms;
  if (grid == 0) return;
  gemm_mxfp8_kernel<<<grid, kThreads, XCfg::SMEM_BYTES, stream>>>(tA, tB, tC, static_cast<const uint8_t*>(sfa),
                                                                   static_cast<const uint8_t*>(sfb), M, N, K, status);
  MT_CUDA_CHECK(cudaGetLastError());
}

}  // namespace mt
