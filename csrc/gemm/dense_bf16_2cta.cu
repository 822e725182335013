// Dense bf16 GEMM on CTA pairs (tcgen05 cta_group::2):  C[M,N] (+)= op(A) * op(B), fp32 accumulation, bf16 or fp32
// out, each operand K-major or MN-major, optional split-K with the accumulating (TMA reduce-add) epilogue.
//
// Two CTAs of a 2-CTA cluster (two SMs of one TPC) work on one 256x256 output tile.  Each CTA stages its own 128
// rows of A and its own 128 columns of B per k-block (32 KB per stage instead of the 48 KB a lone CTA needs for a
// 128x256 tile, so the ring is six deep and the L2 -> shared-memory traffic per FLOP drops by a third); one thread of
// the leader CTA issues tcgen05.mma.cta_group::2 (M = 256, N = 256, K = 16), which reads A from each CTA's own
// shared memory and the two halves of B from both, and accumulates 128 rows x 256 columns into each CTA's own
// tensor memory.  Protocol:
//   * both producers wait on their own `empty` barrier and issue TMA loads whose completion bytes land on the
//     LEADER's `full` barrier (cta_group::2 load form with the peer bit of the barrier address cleared);
//     the leader's producer posts the expected byte count of both CTAs;
//   * the leader's MMA thread waits on `full`, issues the MMAs, and commits with a cluster-wide arrive on both CTAs'
//     `empty` barriers (tcgen05.commit .multicast::cluster: an mbarrier arrive, not a data multicast) and, after
//     the last k-block, on both CTAs' `tmem_full`;
//   * the epilogue warps of both CTAs drain their own TMEM half and arrive on the leader's `tmem_empty` (remote
//     mbarrier arrive for the follower).
// No TMA load uses multicast.  Every wait is bounded; the only unbounded synchronisation is the pair of cluster
// barriers at start and end, which every thread reaches on every path.
#include "../common/ptx.cuh"
#include "../common/tmap.h"
#include "../common/pair.cuh"
#include "../api.h"

namespace mt {
namespace {

constexpr int BM = 128;        // rows per CTA (256 per pair)
constexpr int BN = 256;        // columns per pair tile; each CTA stages BN/2 columns of B
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int kEpiWarps = 4;
constexpr int kThreads = 32 * (2 + kEpiWarps);
constexpr int kEpiStageBytes = 4096;
constexpr int kStages = 6;

struct PCfg {
  static constexpr int A_BYTES = BM * BK * 2;           // 16 KB
  static constexpr int B_BYTES = (BN / 2) * BK * 2;     // 16 KB
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int EPI_BYTES = kEpiWarps * 2 * kEpiStageBytes;
  static constexpr int OFF_EPI = kStages * STAGE_BYTES;
  static constexpr int OFF_BAR = OFF_EPI + EPI_BYTES;
  static constexpr int SMEM_BYTES = OFF_BAR + 256;
  static constexpr int TMEM_COLS = 2 * BN;
  static_assert(SMEM_BYTES <= 232448, "shared memory budget");
};

// Pair-tile order: groups of 8 column tiles, rows fastest inside a group.
__device__ __forceinline__ void tile_coord(int tile, int num_m, int num_n, int& m_idx, int& n_idx) {
  const int per_group = 8 * num_m;
  const int group = tile / per_group;
  const int first_n = group * 8;
  const int gsize = min(8, num_n - first_n);
  const int local = tile - group * per_group;
  m_idx = local / gsize;
  n_idx = first_n + local % gsize;
}

template <bool A_MN, bool B_MN, bool OUT_F32>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
gemm_bf16_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                      const __grid_constant__ CUtensorMap tmC, int M, int N, int K, int accumulate, int splits,
                      int* status) {
  using C = PCfg;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* epi_base = smem + C::OFF_EPI;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::OFF_BAR);
  uint64_t* full_bar = bars;                   // [kStages]  used in the leader only
  uint64_t* empty_bar = bars + kStages;        // [kStages]  one per CTA
  uint64_t* tmem_full = bars + 2 * kStages;    // [2]        one per CTA
  uint64_t* tmem_empty = tmem_full + 2;        // [2]        used in the leader only (8 arrivals)
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
  const int num_items = num_tiles * splits;  // split-K: item = split * num_tiles + tile
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
    prefetch_tmap(&tmB);
    prefetch_tmap(&tmC);
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, C::TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers are initialised before any remote arrive or load completion
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (one per CTA)
    if (lane == 0 && aligned) {
      int it = 0;
      bool ok = true;
      for (int item = pair; item < num_items && ok; item += num_pairs) {
        const int split = item / num_tiles;
        int m_idx, n_idx;
        tile_coord(item - split * num_tiles, num_m, num_n, m_idx, n_idx);
        const int row0 = m_idx * (2 * BM) + rank * BM;          // this CTA's rows of A
        const int col0 = n_idx * BN + rank * (BN / 2);          // this CTA's columns of B
        const int kb_lo = static_cast<int>(static_cast<int64_t>(split) * num_kb / splits);
        const int kb_hi = static_cast<int>(static_cast<int64_t>(split + 1) * num_kb / splits);
        for (int kb = kb_lo; kb < kb_hi; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1;
          if (!mbar_wait(&empty_bar[s], ph ^ 1, abort_flag, status, MT_ERR_TIMEOUT_EMPTY)) {
            ok = false;
            break;
          }
          uint8_t* a_dst = smem + s * C::STAGE_BYTES;
          uint8_t* b_dst = a_dst + C::A_BYTES;
          if (leader) mbar_expect_tx(&full_bar[s], 2 * C::STAGE_BYTES);  // bytes of both CTAs
          const int k0 = kb * BK;
          if constexpr (A_MN) {
#pragma unroll
            for (int a = 0; a < BM / 64; ++a) tma_load_2d_pair(a_dst + a * (BK * 128), &tmA, &full_bar[s], row0 + a * 64, k0);
          } else {
            tma_load_2d_pair(a_dst, &tmA, &full_bar[s], k0, row0);
          }
          if constexpr (B_MN) {
#pragma unroll
            for (int a = 0; a < (BN / 2) / 64; ++a)
              tma_load_2d_pair(b_dst + a * (BK * 128), &tmB, &full_bar[s], col0 + a * 64, k0);
          } else {
            tma_load_2d_pair(b_dst, &tmB, &full_bar[s], k0, col0);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader CTA only)
    if (lane == 0 && leader && aligned) {
      constexpr uint32_t idesc = make_idesc_bf16(2 * BM, BN, A_MN, B_MN);
      int it = 0, tcount = 0;
      bool ok = true;
      for (int item = pair; item < num_items && ok; item += num_pairs, ++tcount) {
        const int split = item / num_tiles;
        const int kb_lo = static_cast<int>(static_cast<int64_t>(split) * num_kb / splits);
        const int kb_hi = static_cast<int>(static_cast<int64_t>(split + 1) * num_kb / splits);
        const int buf = tcount & 1;
        if (!mbar_wait(&tmem_empty[buf], ((tcount >> 1) & 1) ^ 1, abort_flag, status, MT_ERR_TIMEOUT_TMEM_EMPTY)) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + buf * BN;
        for (int kb = kb_lo; kb < kb_hi; ++kb, ++it) {
          const int s = it % kStages;
          if (!mbar_wait(&full_bar[s], (it / kStages) & 1, abort_flag, status, MT_ERR_TIMEOUT_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(smem + s * C::STAGE_BYTES);
          const uint32_t b_addr = a_addr + C::A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t da = A_MN ? make_smem_desc_sw128(a_addr + k * (UMMA_K * 128), BK * 128, 1024)
                                     : make_smem_desc_sw128(a_addr + k * (UMMA_K * 2), 16, 1024);
            const uint64_t db = B_MN ? make_smem_desc_sw128(b_addr + k * (UMMA_K * 128), BK * 128, 1024)
                                     : make_smem_desc_sw128(b_addr + k * (UMMA_K * 2), 16, 1024);
            tc_mma_f16_pair(d_tmem, da, db, idesc, ((kb - kb_lo) | k) != 0 ? 1u : 0u);
          }
          tc_commit_pair(&empty_bar[s]);  // both CTAs' slots reusable once these MMAs have read them
        }
        if (ok) tc_commit_pair(&tmem_full[buf]);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (both CTAs, own 128 rows)
    const int q = warp & 3;
    constexpr int COLS = OUT_F32 ? 32 : 64;  // columns per 128-byte staging row
    uint8_t* stage0 = epi_base + (warp - 2) * 2 * kEpiStageBytes;
    int tcount = 0, nstores = 0;
    for (int item = pair; item < num_items && aligned; item += num_pairs, ++tcount) {
      int m_idx, n_idx;
      tile_coord(item % num_tiles, num_m, num_n, m_idx, n_idx);
      const int buf = tcount & 1;
      if (!mbar_wait_warp(&tmem_full[buf], (tcount >> 1) & 1, abort_flag, status, MT_ERR_TIMEOUT_TMEM_FULL)) break;
      tc_fence_after_sync();
      const int row0 = m_idx * (2 * BM) + rank * BM + q * 32;
      const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * BN;
      for (int c = 0; c < BN / COLS; ++c) {
        const int col0 = n_idx * BN + c * COLS;
        if (col0 >= N) break;
        uint8_t* sbuf = stage0 + (nstores & 1) * kEpiStageBytes;
        if (lane == 0) tma_wait_group_read<1>();
        __syncwarp();
        uint8_t* srow = sbuf + lane * 128;
        if constexpr (OUT_F32) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(t_lane + c * 32, r);
          tc_wait_ld();
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            uint4 v = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
            *reinterpret_cast<uint4*>(srow + ((j ^ (lane & 7)) << 4)) = v;
          }
        } else {
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
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          if (row0 < M) {
            if (accumulate) tma_reduce_add_2d(&tmC, sbuf, col0, row0);
            else tma_store_2d(&tmC, sbuf, col0, row0);
          }
          tma_commit_group();
        }
        ++nstores;
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_leader(&tmem_empty[buf]);  // this warp has drained its part of the accumulator
    }
    if (lane == 0) tma_wait_group<0>();
  }

  // ---------------------------------------------------------------- teardown
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // the peer may still be signalling this CTA's barriers or reading its shared memory
  if (warp == 1) {
    tc_fence_after_sync();
    __syncwarp();
    tmem_dealloc_pair(tmem_base, C::TMEM_COLS);
  }
}

template <bool A_MN, bool B_MN, bool OUT_F32>
void launch_pair(const CUtensorMap& tA, const CUtensorMap& tB, const CUtensorMap& tC, int M, int N, int K, bool accumulate,
                 int* status, int num_sms, cudaStream_t stream) {
  auto kern = gemm_bf16_pair_kernel<A_MN, B_MN, OUT_F32>;
  static bool configured = false;
  if (!configured) {
    MT_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, PCfg::SMEM_BYTES));
    configured = true;
  }
  const int tiles = ((M + 2 * BM - 1) / (2 * BM)) * ((N + BN - 1) / BN);
  const int max_pairs = num_sms / 2;
  // split K when the pair tiles fill the last wave badly and the epilogue adds into C anyway (weight gradients)
  int splits = 1;
  if (OUT_F32 && accumulate) {
    const int num_kb = (K + BK - 1) / BK;
    auto eff = [&](int sp) {
      const int items = tiles * sp;
      return static_cast<double>(items) / (static_cast<double>((items + max_pairs - 1) / max_pairs) * max_pairs);
    };
    double best = eff(1);
    for (int sp = 2; sp <= 6; ++sp) {
      if (num_kb / sp < 16) break;
      if (eff(sp) > best + 0.08) {
        best = eff(sp);
        splits = sp;
      }
    }
  }
  const int items = tiles * splits;
  const int pairs = items < max_pairs ? items : max_pairs;
  kern<<<2 * pairs, kThreads, PCfg::SMEM_BYTES, stream>>>(tA, tB, tC, M, N, K, accumulate ? 1 : 0, splits, status);
  MT_CUDA_CHECK(cudaGetLastError());
}

}  // namespace

// A: K-major [M,K] or MN-major [K,M] (row pitch lda); B: K-major [N,K] or MN-major [K,N] (ldb); C: [M,N] (ldc), bf16
// or fp32; accumulate -> C += result (TMA element-wise add).
void gemm_bf16_pair(const void* A, const void* B, void* Cout, int M, int N, int K, int64_t lda, int64_t ldb, int64_t ldc,
                    bool a_mn_major, bool b_mn_major, bool out_f32, bool accumulate, int* status, int num_sms,
                    cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return;
  const auto bf = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const auto sw = CU_TENSOR_MAP_SWIZZLE_128B;
  CUtensorMap tA = a_mn_major ? make_tmap_2d(A, bf, 2, K, M, lda, BK, 64, sw) : make_tmap_2d(A, bf, 2, M, K, lda, BM, BK, sw);
  CUtensorMap tB = b_mn_major ? make_tmap_2d(B, bf, 2, K, N, ldb, BK, 64, sw) : make_tmap_2d(B, bf, 2, N, K, ldb, BN / 2, BK, sw);
  CUtensorMap tC = out_f32 ? make_tmap_2d(Cout, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, M, N, ldc, 32, 32, sw)
                           : make_tmap_2d(Cout, bf, 2, M, N, ldc, 32, 64, sw);
#define MT_PAIR_CASE(AM, BMJ, F32)                                \
  if (a_mn_major == AM && b_mn_major == BMJ && out_f32 == F32)    \
    return launch_pair<AM, BMJ, F32>(tA, tB, tC, M, N, K, accumulate, status, num_sms, stream);
  MT_PAIR_CASE(false, false, false)
  MT_PAIR_CASE(false, true, false)
  MT_PAIR_CASE(true, false, false)
  MT_PAIR_CASE(true, true, false)
  MT_PAIR_CASE(false, false, true)
  MT_PAIR_CASE(false, true, true)
  MT_PAIR_CASE(true, false, true)
  MT_PAIR_CASE(true, true, true)
#undef MT_PAIR_CASE
}

}  // namespace mt
