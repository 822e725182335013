// Grouped (per-expert) bf16 GEMMs on CTA pairs (tcgen05 cta_group::2): the MoE counterpart of dense_bf16_2cta.cu.
//
// A pair works on a 256-row x 256-column output tile; each CTA stages its own 128 rows of A and 128 columns of B
// (six-stage ring), the leader issues the M = 256 MMAs, both CTAs drain their own half of the accumulator.
//   MODE_FWD   Y[rows, N] = X[rows, K] * W[e].  Experts are padded to multiples of 128 rows, so an expert may hold
//              an odd number of 128-row blocks: its last pair tile then has only the leader's half inside the
//              expert; the follower still feeds the pair MMA (with rows of whatever follows) but stores nothing.
//              Tiles are enumerated per expert through a prefix sum of ceil(blocks / 2) built in shared memory.
//   MODE_WGRAD dW[e][K, N] (+)= X_e^T * G_e with 256 x 256 tiles of dW[e]; contraction over the expert's rows.
//   SCATTER    (forward only) the epilogue does not store the tile: every output row is written, 128 contiguous bytes
//              per group of eight lanes, to the address `row_dst[row]` - a row of a buffer in another GPU's (or this
//              GPU's) memory - and rows whose entry is 0 (padding) are dropped.  This is the expert GEMM fused with
//              the combine (or dispatch-gradient) all-to-all of expert parallelism: the rows travel over NVLink while
//              later tiles are still being multiplied.  Plain peer stores; the consumer reads after a barrier.
// Barrier protocol, bounded waits and the absence of multicast loads are as in the dense pair kernel.
#include "../common/ptx.cuh"
#include "../common/tmap.h"
#include "../common/pair.cuh"
#include "../api.h"

namespace mt {
namespace {

constexpr int BM = 128;   // rows per CTA (256 per pair)
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int kEpiWarps = 4;
constexpr int kThreads = 32 * (2 + kEpiWarps);
constexpr int kEpiStageBytes = 4096;
constexpr int kStages = 6;
constexpr int kMaxExperts = 256;  // more experts than this per rank take the single-CTA kernel

struct GPCfg {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = (BN / 2) * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int EPI_BYTES = kEpiWarps * 2 * kEpiStageBytes;
  static constexpr int OFF_EPI = kStages * STAGE_BYTES;
  static constexpr int OFF_BAR = OFF_EPI + EPI_BYTES;
  static constexpr int OFF_OFFS = OFF_BAR + 256;
  static constexpr int SMEM_BYTES = OFF_OFFS + 2 * (kMaxExperts + 1) * 4;
  static constexpr int TMEM_COLS = 2 * BN;
  static_assert(SMEM_BYTES <= 232448, "shared memory budget");
};

struct Tile {
  int e, row0, n0, kb0, kb1, row_end;  // row_end: first row (fwd) not belonging to the expert
};

enum { MODE_FWD = 0, MODE_WGRAD = 1 };

template <int MODE>
__device__ __forceinline__ Tile decode_tile(int tile, const int* offs, const int* pref, int E, int N, int K) {
  const int num_n = (N + BN - 1) / BN;
  Tile t;
  if (MODE == MODE_FWD) {
    const int pt = tile / num_n;
    t.n0 = (tile % num_n) * BN;
    int lo = 0, hi = E;  // largest e with pref[e] <= pt
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (pref[mid] <= pt) lo = mid;
      else hi = mid;
    }
    t.e = lo;
    t.row0 = offs[lo] + (pt - pref[lo]) * (2 * BM);
    t.row_end = offs[lo + 1];
    t.kb0 = 0;
    t.kb1 = (K + BK - 1) / BK;
  } else {
    const int num_kt = (K + 2 * BM - 1) / (2 * BM);
    t.e = tile / (num_kt * num_n);
    const int rem = tile % (num_kt * num_n);
    t.row0 = (rem / num_n) * (2 * BM);
    t.n0 = (rem % num_n) * BN;
    t.kb0 = offs[t.e] / BK;
    t.kb1 = offs[t.e + 1] / BK;
    t.row_end = K;
  }
  return t;
}

template <int MODE, bool B_MN, bool OUT_F32, bool SCATTER = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
grouped_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const __grid_constant__ CUtensorMap tmC, const int* __restrict__ offsets, int E, int N, int K,
                    int accumulate, int* status, const unsigned long long* __restrict__ row_dst = nullptr) {
  static_assert(!SCATTER || (MODE == MODE_FWD && !OUT_F32), "row scatter is a forward, bf16 epilogue");
  using C = GPCfg;
  constexpr bool A_MN = (MODE == MODE_WGRAD);
  constexpr bool BMN = (MODE == MODE_WGRAD) ? true : B_MN;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* epi_base = smem + C::OFF_EPI;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::OFF_BAR);
  uint64_t* full_bar = bars;                   // leader only
  uint64_t* empty_bar = bars + kStages;        // per CTA
  uint64_t* tmem_full = bars + 2 * kStages;    // per CTA
  uint64_t* tmem_empty = tmem_full + 2;        // leader only (8 arrivals)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* offs = reinterpret_cast<int*>(smem + C::OFF_OFFS);
  int* pref = offs + (kMaxExperts + 1);  // pair tiles of the experts before e (forward mode)

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  const bool aligned = (smem_u32(smem) & 1023u) == 0;

  for (int i = threadIdx.x; i <= E; i += blockDim.x) offs[i] = offsets[i];
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
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int e = 0; e < E; ++e) {
      pref[e] = run;
      run += (offs[e + 1] - offs[e] + 2 * BM - 1) / (2 * BM);
    }
    pref[E] = run;
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const int num_n = (N + BN - 1) / BN;
  const int num_tiles = (MODE == MODE_FWD) ? pref[E] * num_n : E * ((K + 2 * BM - 1) / (2 * BM)) * num_n;

  if (warp == 0) {
    if (lane == 0 && aligned) {
      int it = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        const Tile t = decode_tile<MODE>(tile, offs, pref, E, N, K);
        const int row0 = t.row0 + rank * BM;
        const int col0 = t.n0 + rank * (BN / 2);
        for (int kb = t.kb0; kb < t.kb1; ++kb, ++it) {
          const int s = it % kStages;
          if (!mbar_wait(&empty_bar[s], ((it / kStages) & 1) ^ 1, abort_flag, status, MT_ERR_TIMEOUT_EMPTY)) { ok = false; break; }
          uint8_t* a_dst = smem + s * C::STAGE_BYTES;
          uint8_t* b_dst = a_dst + C::A_BYTES;
          if (leader) mbar_expect_tx(&full_bar[s], 2 * C::STAGE_BYTES);
          const int k0 = kb * BK;
          if (MODE == MODE_FWD) {
            tma_load_2d_pair(a_dst, &tmA, &full_bar[s], k0, row0);
            if (BMN) {
#pragma unroll
              for (int a = 0; a < (BN / 2) / 64; ++a)
                tma_load_3d_pair(b_dst + a * (BK * 128), &tmB, &full_bar[s], col0 + a * 64, k0, t.e);
            } else {
              tma_load_3d_pair(b_dst, &tmB, &full_bar[s], k0, col0, t.e);
            }
          } else {
#pragma unroll
            for (int a = 0; a < BM / 64; ++a) tma_load_2d_pair(a_dst + a * (BK * 128), &tmA, &full_bar[s], row0 + a * 64, k0);
#pragma unroll
            for (int a = 0; a < (BN / 2) / 64; ++a)
              tma_load_2d_pair(b_dst + a * (BK * 128), &tmB, &full_bar[s], col0 + a * 64, k0);
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && leader && aligned) {
      constexpr uint32_t idesc = make_idesc_bf16(2 * BM, BN, A_MN, BMN);
      int it = 0, tcount = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        const Tile t = decode_tile<MODE>(tile, offs, pref, E, N, K);
        if (t.kb1 <= t.kb0) continue;  // empty expert (weight-gradient mode): nothing to accumulate
        const int buf = tcount & 1;
        if (!mbar_wait(&tmem_empty[buf], ((tcount >> 1) & 1) ^ 1, abort_flag, status, MT_ERR_TIMEOUT_TMEM_EMPTY)) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + buf * BN;
        for (int kb = t.kb0; kb < t.kb1; ++kb, ++it) {
          const int s = it % kStages;
          if (!mbar_wait(&full_bar[s], (it / kStages) & 1, abort_flag, status, MT_ERR_TIMEOUT_FULL)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(smem + s * C::STAGE_BYTES);
          const uint32_t b_addr = a_addr + C::A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t da = A_MN ? make_smem_desc_sw128(a_addr + k * (UMMA_K * 128), BK * 128, 1024)
                                     : make_smem_desc_sw128(a_addr + k * (UMMA_K * 2), 16, 1024);
            const uint64_t db = BMN ? make_smem_desc_sw128(b_addr + k * (UMMA_K * 128), BK * 128, 1024)
                                    : make_smem_desc_sw128(b_addr + k * (UMMA_K * 2), 16, 1024);
            tc_mma_f16_pair(d_tmem, da, db, idesc, (kb > t.kb0 || k != 0) ? 1u : 0u);
          }
          tc_commit_pair(&empty_bar[s]);
        }
        if (ok) tc_commit_pair(&tmem_full[buf]);
        ++tcount;
      }
    }
  } else {
    const int q = warp & 3;
    constexpr int COLS = OUT_F32 ? 32 : 64;
    uint8_t* stage0 = epi_base + (warp - 2) * 2 * kEpiStageBytes;
    int tcount = 0, nstores = 0;
    for (int tile = pair; tile < num_tiles && aligned; tile += num_pairs) {
      const Tile t = decode_tile<MODE>(tile, offs, pref, E, N, K);
      if (t.kb1 <= t.kb0) continue;
      const int buf = tcount & 1;
      if (!mbar_wait_warp(&tmem_full[buf], (tcount >> 1) & 1, abort_flag, status, MT_ERR_TIMEOUT_TMEM_FULL)) break;
      tc_fence_after_sync();
      const int row0 = t.row0 + rank * BM + q * 32;
      const bool rows_live = row0 < t.row_end;  // forward: the follower's half may lie beyond the expert's rows
      const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * BN;
      unsigned long long my_dst = 0;  // SCATTER: lane l holds the destination of row row0 + l
      if constexpr (SCATTER) {
        if (rows_live) my_dst = row_dst[row0 + lane];
      }
      for (int c = 0; c < BN / COLS && rows_live; ++c) {
        const int col0 = t.n0 + c * COLS;
        if (col0 >= N) break;
        uint8_t* sbuf = stage0 + (nstores & 1) * kEpiStageBytes;
        if constexpr (!SCATTER) {
          if (lane == 0) tma_wait_group_read<1>();
        }
        __syncwarp();
        uint8_t* srow = sbuf + lane * 128;
        if constexpr (OUT_F32) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(t_lane + c * 32, r);
          tc_wait_ld();
#pragma unroll
          for (int j = 0; j < 8; ++j)
            *reinterpret_cast<uint4*>(srow + ((j ^ (lane & 7)) << 4)) =
                make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
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
        if constexpr (SCATTER) {
          __syncwarp();
          // read the staged 32 x 128-byte chunk back row-wise: eight lanes carry one row's 128 contiguous bytes
          const int ch = lane & 7;
          const bool col_ok = col0 + ch * 8 < N;
#pragma unroll
          for (int it = 0; it < 8; ++it) {
            const int rr = it * 4 + (lane >> 3);
            const unsigned long long dst = __shfl_sync(0xffffffffu, my_dst, rr);
            const uint4 v = *reinterpret_cast<const uint4*>(sbuf + rr * 128 + ((ch ^ (rr & 7)) << 4));
            if (dst != 0 && col_ok)
              *reinterpret_cast<uint4*>(dst + static_cast<unsigned long long>(col0 + ch * 8) * 2) = v;
          }
        } else {
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            if (MODE == MODE_FWD) tma_store_2d(&tmC, sbuf, col0, row0);
            else if (accumulate) tma_reduce_add_3d(&tmC, sbuf, col0, row0, t.e);
            else tma_store_3d(&tmC, sbuf, col0, row0, t.e);
            tma_commit_group();
          }
        }
        ++nstores;
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_leader(&tmem_empty[buf]);
      ++tcount;
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

template <typename Kern>
void configure(Kern k) {
  MT_CUDA_CHECK(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, GPCfg::SMEM_BYTES));
}

}  // namespace

void grouped_gemm_bf16_pair(const void* X, const void* W, void* Y, const int* offsets, int E, int M_cap, int N, int K,
                            bool w_mn_major, int* status, int num_sms, cudaStream_t stream) {
  if (M_cap <= 0 || E <= 0) return;
  if (E > kMaxExperts) throw std::runtime_error("grouped_gemm_bf16_pair: too many experts");
  const auto bf = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const auto sw = CU_TENSOR_MAP_SWIZZLE_128B;
  CUtensorMap tA = make_tmap_2d(X, bf, 2, M_cap, K, K, BM, BK, sw);
  CUtensorMap tB = w_mn_major ? make_tmap_3d(W, bf, 2, E, K, N, (uint64_t)K * N, N, 1, BK, 64, sw)
                              : make_tmap_3d(W, bf, 2, E, N, K, (uint64_t)N * K, K, 1, BN / 2, BK, sw);
  CUtensorMap tC = make_tmap_2d(Y, bf, 2, M_cap, N, N, 32, 64, sw);
  static bool configured = false;
  if (!configured) {
    configure(grouped_pair_kernel<MODE_FWD, true, false>);
    configure(grouped_pair_kernel<MODE_FWD, false, false>);
    configured = true;
  }
  const int grid = (num_sms / 2) * 2;
  if (w_mn_major)
    grouped_pair_kernel<MODE_FWD, true, false><<<grid, kThreads, GPCfg::SMEM_BYTES, stream>>>(tA, tB, tC, offsets, E, N, K, 0, status);
  else
    grouped_pair_kernel<MODE_FWD, false, false><<<grid, kThreads, GPCfg::SMEM_BYTES, stream>>>(tA, tB, tC, offsets, E, N, K, 0, status);
  MT_CUDA_CHECK(cudaGetLastError());
}

// Same product, but output row r is written to the address row_dst[r] (0 = drop the row) instead of Y; the addresses
// may point into peer-mapped memory of other GPUs.  `row_dst` has M_cap entries; every destination row holds N bf16.
void grouped_gemm_scatter_bf16_pair(const void* X, const void* W, const unsigned long long* row_dst, const int* offsets,
                                    int E, int M_cap, int N, int K, bool w_mn_major, int* status, int num_sms,
                                    cudaStream_t stream) {
  if (M_cap <= 0 || E <= 0) return;
  if (E > kMaxExperts) throw std::runtime_error("grouped_gemm_scatter_bf16_pair: too many experts");
  if (N % 8 != 0) throw std::runtime_error("grouped_gemm_scatter_bf16_pair: N must be a multiple of 8");
  const auto bf = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const auto sw = CU_TENSOR_MAP_SWIZZLE_128B;
  CUtensorMap tA = make_tmap_2d(X, bf, 2, M_cap, K, K, BM, BK, sw);
  CUtensorMap tB = w_mn_major ? make_tmap_3d(W, bf, 2, E, K, N, (uint64_t)K * N, N, 1, BK, 64, sw)
                              : make_tmap_3d(W, bf, 2, E, N, K, (uint64_t)N * K, K, 1, BN / 2, BK, sw);
  static bool configured = false;
  if (!configured) {
    configure(grouped_pair_kernel<MODE_FWD, true, false, true>);
    configure(grouped_pair_kernel<MODE_FWD, false, false, true>);
    configured = true;
  }
  const int grid = (num_sms / 2) * 2;
  if (w_mn_major)
    grouped_pair_kernel<MODE_FWD, true, false, true><<<grid, kThreads, GPCfg::SMEM_BYTES, stream>>>(tA, tB, tA, offsets, E, N, K, 0, status, row_dst);
  else
    grouped_pair_kernel<MODE_FWD, false, false, true><<<grid, kThreads, GPCfg::SMEM_BYTES, stream>>>(tA, tB, tA, offsets, E, N, K, 0, status, row_dst);
  MT_CUDA_CHECK(cudaGetLastError());
}

void grouped_wgrad_bf16_pair(const void* X, const void* G, void* dW, const int* offsets, int E, int M_cap, int N, int K,
                             bool out_f32, bool accumulate, int* status, int num_sms, cudaStream_t stream) {
  if (M_cap <= 0 || E <= 0) return;
  if (E > kMaxExperts) throw std::runtime_error("grouped_wgrad_bf16_pair: too many experts");
  const auto bf = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const auto sw = CU_TENSOR_MAP_SWIZZLE_128B;
  CUtensorMap tA = make_tmap_2d(X, bf, 2, M_cap, K, K, BK, 64, sw);
  CUtensorMap tB = make_tmap_2d(G, bf, 2, M_cap, N, N, BK, 64, sw);
  CUtensorMap tC = out_f32 ? make_tmap_3d(dW, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, E, K, N, (uint64_t)K * N, N, 1, 32, 32, sw)
                           : make_tmap_3d(dW, bf, 2, E, K, N, (uint64_t)K * N, N, 1, 32, 64, sw);
  static bool configured = false;
  if (!configured) {
    configure(grouped_pair_kernel<MODE_WGRAD, true, true>);
    configure(grouped_pair_kernel<MODE_WGRAD, true, false>);
    configured = true;
  }
  const int grid = (num_sms / 2) * 2;
  if (out_f32)
    grouped_pair_kernel<MODE_WGRAD, true, true><<<grid, kThreads, GPCfg::SMEM_BYTES, stream>>>(tA, tB, tC, offsets, E, N, K, accumulate ? 1 : 0, status);
  else
    grouped_pair_kernel<MODE_WGRAD, true, false><<<grid, kThreads, GPCfg::SMEM_BYTES, stream>>>(tA, tB, tC, offsets, E, N, K, accumulate ? 1 : 0, status);
  MT_CUDA_CHECK(cudaGetLastError());
}

}  // namespace mt
