// Gated-MLP front half as ONE GEMM on CTA pairs (tcgen05 cta_group::2):
//     G = X Wg,  U = X Wu,  H = act(G) * U        X [T, K] bf16, Wg / Wu [K, I] bf16 (as the parameters are stored)
// The pair works on 256 rows x 128 output columns: the leader CTA stages the 128 columns of Wg, the follower the
// same 128 columns of Wu, so the M = 256, N = 256 pair MMA leaves [gate | up] for identical output columns side by
// side in each CTA's accumulator.  The epilogue stores G and U (the backward pass needs them) into the halves of one
// [T, 2I] buffer and H = act(G) * U into [T, I] - the separate activation kernel and its re-read of G and U are gone
// (mintext/modules/linear.py:218-225 for the layer semantics).  Ring, barriers, bounded waits and the absence of
// multicast loads are those of dense_bf16_2cta.cu.
#include "../common/ptx.cuh"
#include "../common/tmap.h"
#include "../common/pair.cuh"
#include "../api.h"

namespace mt {
namespace {

constexpr int BM = 128;        // rows per CTA (256 per pair)
constexpr int BN = 256;        // accumulator columns per CTA: 128 gate + 128 up
constexpr int BO = 128;        // output columns per pair tile
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int kEpiWarps = 4;
constexpr int kThreads = 32 * (2 + kEpiWarps);
constexpr int kEpiStageBytes = 4096;
constexpr int kStages = 6;

struct GCfg {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BO * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
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

// ACT: 0 silu, 1 gelu (tanh approximation), 2 gelu (erf), 3 relu - the codes of the stand-alone activation kernel
template <int ACT>
__device__ __forceinline__ float act_fn(float x) {
  if (ACT == 0) return x / (1.f + __expf(-x));
  if (ACT == 1) {
    const float k0 = 0.7978845608028654f, k1 = 0.044715f;
    return 0.5f * x * (1.f + tanhf(k0 * (x + k1 * x * x * x)));
  }
  if (ACT == 2) return 0.5f * x * (1.f + erff(x * 0.7071067811865476f));
  return x > 0.f ? x : 0.f;
}

template <int ACT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
gemm_gated_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmBg,
                       const __grid_constant__ CUtensorMap tmBu, const __grid_constant__ CUtensorMap tmGU,
                       const __grid_constant__ CUtensorMap tmH, int T, int I, int K, int* status) {
  using C = GCfg;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* epi_base = smem + C::OFF_EPI;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::OFF_BAR);
  uint64_t* full_bar = bars;                   // leader only
  uint64_t* empty_bar = bars + kStages;        // per CTA
  uint64_t* tmem_full = bars + 2 * kStages;    // per CTA
  uint64_t* tmem_empty = tmem_full + 2;        // leader only (8 arrivals)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  const int num_m = (T + 2 * BM - 1) / (2 * BM);
  const int num_n = I / BO;
  const int num_tiles = num_m * num_n;
  const int num_kb = (K + BK - 1) / BK;
  const bool aligned = (smem_u32(smem) & 1023u) == 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
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
    prefetch_tmap(leader ? &tmBg : &tmBu);
    prefetch_tmap(&tmGU);
    prefetch_tmap(&tmH);
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
    // ------------------------------------------------------------ TMA producer (one per CTA)
    if (lane == 0 && aligned) {
      const CUtensorMap* tmB = leader ? &tmBg : &tmBu;  // the leader's half of B is gate, the follower's is up
      int it = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        int m_idx, n_idx;
        tile_coord(tile, num_m, num_n, m_idx, n_idx);
        const int row0 = m_idx * (2 * BM) + rank * BM;
        const int col0 = n_idx * BO;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % kStages;
          if (!mbar_wait(&empty_bar[s], ((it / kStages) & 1) ^ 1, abort_flag, status, MT_ERR_TIMEOUT_EMPTY)) {
            ok = false;
            break;
          }
          uint8_t* a_dst = smem + s * C::STAGE_BYTES;
          uint8_t* b_dst = a_dst + C::A_BYTES;
          if (leader) mbar_expect_tx(&full_bar[s], 2 * C::STAGE_BYTES);
          const int k0 = kb * BK;
          tma_load_2d_pair(a_dst, &tmA, &full_bar[s], k0, row0);
#pragma unroll
          for (int a = 0; a < BO / 64; ++a) tma_load_2d_pair(b_dst + a * (BK * 128), tmB, &full_bar[s], col0 + a * 64, k0);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader CTA only)
    if (lane == 0 && leader && aligned) {
      constexpr uint32_t idesc = make_idesc_bf16(2 * BM, BN, false, true);
      int it = 0, tcount = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, ++tcount) {
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
          const uint64_t da = make_smem_desc_sw128(a_addr, 16, 1024);
          const uint64_t db = make_smem_desc_sw128(b_addr, BK * 128, 1024);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            tc_mma_f16_pair(d_tmem, da + k * ((UMMA_K * 2) >> 4), db + k * ((UMMA_K * 128) >> 4), idesc,
                            (kb | k) != 0 ? 1u : 0u);
          tc_commit_pair(&empty_bar[s]);
        }
        if (ok) tc_commit_pair(&tmem_full[buf]);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (both CTAs, own 128 rows)
    // Accumulator columns [0, 128) are gate, [128, 256) up, for output columns n_idx * 128 ...  Three boxes of 32 rows
    // x 64 columns leave per 64-column group: G and U into the halves of the [T, 2I] buffer, H into [T, I].
    const int q = warp & 3;
    uint8_t* stage0 = epi_base + (warp - 2) * 2 * kEpiStageBytes;
    int tcount = 0, nstores = 0;
    auto stage_store = [&](const CUtensorMap* map, const uint32_t (&lo)[32], const uint32_t (&hi)[32], int col, int row) {
      // lo / hi: 32 + 32 columns of one 64-column box, as fp32 bit patterns
      uint8_t* sbuf = stage0 + (nstores & 1) * kEpiStageBytes;
      if (lane == 0) tma_wait_group_read<1>();
      __syncwarp();
      uint8_t* srow = sbuf + lane * 128;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const uint32_t (&r)[32] = h == 0 ? lo : hi;
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
        if (row < T) tma_store_2d(map, sbuf, col, row);
        tma_commit_group();
      }
      ++nstores;
    };
    for (int tile = pair; tile < num_tiles && aligned; tile += num_pairs, ++tcount) {
      int m_idx, n_idx;
      tile_coord(tile, num_m, num_n, m_idx, n_idx);
      const int buf = tcount & 1;
      if (!mbar_wait_warp(&tmem_full[buf], (tcount >> 1) & 1, abort_flag, status, MT_ERR_TIMEOUT_TMEM_FULL)) break;
      tc_fence_after_sync();
      const int row0 = m_idx * (2 * BM) + rank * BM + q * 32;
      const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * BN;
#pragma unroll 1
      for (int c = 0; c < BO / 64; ++c) {
        const int col0 = n_idx * BO + c * 64;
        uint32_t g0[32], g1[32], u0[32], u1[32];
        tmem_ld_32x32b_x32(t_lane + c * 64, g0);
        tmem_ld_32x32b_x32(t_lane + c * 64 + 32, g1);
        tc_wait_ld();
        stage_store(&tmGU, g0, g1, col0, row0);
        tmem_ld_32x32b_x32(t_lane + BO + c * 64, u0);
        tmem_ld_32x32b_x32(t_lane + BO + c * 64 + 32, u1);
        tc_wait_ld();
        stage_store(&tmGU, u0, u1, I + col0, row0);
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          g0[e] = __float_as_uint(act_fn<ACT>(__uint_as_float(g0[e])) * __uint_as_float(u0[e]));
          g1[e] = __float_as_uint(act_fn<ACT>(__uint_as_float(g1[e])) * __uint_as_float(u1[e]));
        }
        stage_store(&tmH, g0, g1, col0, row0);
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

template <int ACT>
void launch_gated(const CUtensorMap& tA, const CUtensorMap& tBg, const CUtensorMap& tBu, const CUtensorMap& tGU,
                  const CUtensorMap& tH, int T, int I, int K, int* status, int num_sms, cudaStream_t stream) {
  auto kern = gemm_gated_pair_kernel<ACT>;
  static bool configured = false;
  if (!configured) {
    MT_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, GCfg::SMEM_BYTES));
    configured = true;
  }
  const int tiles = ((T + 2 * BM - 1) / (2 * BM)) * (I / BO);
  const int max_pairs = num_sms / 2;
  const int pairs = tiles < max_pairs ? tiles : max_pairs;
  kern<<<2 * pairs, kThreads, GCfg::SMEM_BYTES, stream>>>(tA, tBg, tBu, tGU, tH, T, I, K, status);
  MT_CUDA_CHECK(cudaGetLastError());
}

}  // namespace

// X [T, K] (row pitch ldx); Wg, Wu [K, I] contiguous; GU [T, 2I] and H [T, I] contiguous bf16.  I % 128 == 0.
void gemm_gate_up_act_pair(const void* X, const void* Wg, const void* Wu, void* GU, void* H, int T, int I, int K,
                           int64_t ldx, int act, int* status, int num_sms, cudaStream_t stream) {
  if (T <= 0 || I <= 0 || K <= 0) return;
  if (I % BO != 0 || K % 8 != 0) throw std::runtime_error("gemm_gate_up_act_pair: I must be a multiple of 128, K of 8");
  const auto bf = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const auto sw = CU_TENSOR_MAP_SWIZZLE_128B;
  CUtensorMap tA = make_tmap_2d(X, bf, 2, T, K, ldx, BM, BK, sw);
  CUtensorMap tBg = make_tmap_2d(Wg, bf, 2, K, I, I, BK, 64, sw);
  CUtensorMap tBu = make_tmap_2d(Wu, bf, 2, K, I, I, BK, 64, sw);
  CUtensorMap tGU = make_tmap_2d(GU, bf, 2, T, 2 * I, 2 * I, 32, 64, sw);
  CUtensorMap tH = make_tmap_2d(H, bf, 2, T, I, I, 32, 64, sw);
  switch (act) {
    case 0: return launch_gated<0>(tA, tBg, tBu, tGU, tH, T, I, K, status, num_sms, stream);
    case 1: return launch_gated<1>(tA, tBg, tBu, tGU, tH, T, I, K, status, num_sms, stream);
    case 2: return launch_gated<2>(tA, tBg, tBu, tGU, tH, T, I, K, status, num_sms, stream);
    default: return launch_gated<3>(tA, tBg, tBu, tGU, tH, T, I, K, status, num_sms, stream);
  }
}

}  // namespace mt
