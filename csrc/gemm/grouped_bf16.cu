// Grouped (per-expert) bf16 GEMMs for MoE on sm_100a, same pipeline as the dense kernel (TMA ring -> tcgen05.mma ->
// double-buffered TMEM accumulators -> swizzled smem -> TMA store), with a device-side tile scheduler over groups.
//
// Row layout contract: the rows of X / Y belonging to expert e are offsets[e] .. offsets[e+1], and every offset is a
// multiple of 128 (the dispatch step pads each group with zero rows).  Hence no output tile straddles two experts
// and no contraction block of the weight-gradient product mixes rows of two experts.
//
//   MODE_FWD   Y[rows, N] = X[rows, K] * W[e]        W is [E, K, N] (read MN-major) or, for the data-gradient
//                                                    product dX = dY * W[e]^T, [E, N_out, K_contract] read K-major.
//   MODE_WGRAD dW[e][K, N] (+)= X_e^T * G_e          contraction over the expert's (padded) rows; X, G read MN-major;
//                                                    fp32 or bf16 output through a 3-D tensor map (clipped per expert).
// The number of row tiles is data dependent and read from offsets[E] on the device: no host synchronisation.
#include "../common/ptx.cuh"
#include "../common/tmap.h"
#include "../api.h"
#include <cstdlib>

namespace mt {
namespace {

bool single_cta_only() {  // MT_GEMM_SINGLE_CTA=1 keeps the single-CTA kernels (for comparisons)
  static const bool v = [] {
    const char* e = std::getenv("MT_GEMM_SINGLE_CTA");
    return e != nullptr && e[0] == '1';
  }();
  return v;
}

// Kernel choice of the calling thread for the next grouped launches: 0 = default (CTA pairs unless
// MT_GEMM_SINGLE_CTA=1), 1 = single-CTA 128 x 256 tiles, 2 = CTA-pair 256 x 256 tiles.  The autotuner times both.
thread_local int g_variant = 0;

bool use_pair_kernels() { return g_variant == 2 || (g_variant == 0 && !single_cta_only()); }

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int kEpiWarps = 4;
constexpr int kThreads = 32 * (2 + kEpiWarps);
constexpr int kEpiStageBytes = 4096;
constexpr int kMaxExperts = 640;

struct GCfg {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = 4;
  static constexpr int EPI_BYTES = kEpiWarps * 2 * kEpiStageBytes;
  static constexpr int OFF_BYTES = (kMaxExperts + 1) * 4;
  static constexpr int BAR_BYTES = 256;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + EPI_BYTES + BAR_BYTES + OFF_BYTES;
  static constexpr int TMEM_COLS = 2 * BN;
  static_assert(SMEM_BYTES <= 232448, "shared memory budget");
};

struct Tile {
  int e;        // expert
  int row0;     // fwd: first row of the tile in X / Y ; wgrad: first K index (rows of dW[e])
  int n0;       // first output column
  int kb0, kb1; // contraction blocks (units of BK) ; wgrad: absolute row blocks of the expert
};

enum { MODE_FWD = 0, MODE_WGRAD = 1 };

template <int MODE>
__device__ __forceinline__ int num_tiles_of(const int* offs, int E, int N, int K) {
  const int num_n = (N + BN - 1) / BN;
  if (MODE == MODE_FWD) return (offs[E] / BM) * num_n;
  return E * ((K + BM - 1) / BM) * num_n;
}

template <int MODE>
__device__ __forceinline__ Tile decode_tile(int tile, const int* offs, int E, int N, int K) {
  const int num_n = (N + BN - 1) / BN;
  Tile t;
  if (MODE == MODE_FWD) {
    const int mt = tile / num_n;
    t.n0 = (tile % num_n) * BN;
    t.row0 = mt * BM;
    int lo = 0, hi = E;  // largest e with offs[e] <= row0
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (offs[mid] <= t.row0) lo = mid;
      else hi = mid;
    }
    t.e = lo;
    t.kb0 = 0;
    t.kb1 = (K + BK - 1) / BK;
  } else {
    const int num_kt = (K + BM - 1) / BM;
    t.e = tile / (num_kt * num_n);
    const int rem = tile % (num_kt * num_n);
    t.row0 = (rem / num_n) * BM;
    t.n0 = (rem % num_n) * BN;
    t.kb0 = offs[t.e] / BK;
    t.kb1 = offs[t.e + 1] / BK;
  }
  return t;
}

// FWD: A = X K-major 2-D ; B = W 3-D, B_MN selects [E,K,N] (MN-major) or [E,N,K] (K-major).
// WGRAD: A = X MN-major 2-D ; B = G MN-major 2-D ; C 3-D [E,K,N].
template <int MODE, bool B_MN, bool OUT_F32>
__global__ void __launch_bounds__(kThreads, 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const __grid_constant__ CUtensorMap tmC, const int* __restrict__ offsets, int E, int N, int K,
                    int accumulate, int* status) {
  using C = GCfg;
  constexpr bool A_MN = (MODE == MODE_WGRAD);
  constexpr bool BMN = (MODE == MODE_WGRAD) ? true : B_MN;
  extern __shared__ __align__(1024) uint8_t smem[];
  if ((smem_u32(smem) & 1023u) != 0) {  // swizzled tiles need 1024-byte alignment
    if (threadIdx.x == 0 && status) atomicCAS(status, 0, MT_ERR_BAD_ARGS);
    return;
  }
  uint8_t* epi_base = smem + C::STAGES * C::STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(epi_base + C::EPI_BYTES);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + C::STAGES;
  uint64_t* tmem_full = bars + 2 * C::STAGES;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* offs = reinterpret_cast<int*>(reinterpret_cast<uint8_t*>(bars) + C::BAR_BYTES);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i <= E; i += blockDim.x) offs[i] = offsets[i];
  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) {
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
  const int num_tiles = num_tiles_of<MODE>(offs, E, N, K);

  if (warp == 0) {
    if (lane == 0) {
      int it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const Tile t = decode_tile<MODE>(tile, offs, E, N, K);
        for (int kb = t.kb0; kb < t.kb1; ++kb, ++it) {
          const int s = it % C::STAGES;
          const uint32_t ph = (it / C::STAGES) & 1;
          if (!mbar_wait(&empty_bar[s], ph ^ 1, abort_flag, status, MT_ERR_TIMEOUT_EMPTY)) { ok = false; break; }
          uint8_t* a_dst = smem + s * C::STAGE_BYTES;
          uint8_t* b_dst = a_dst + C::A_BYTES;
          mbar_expect_tx(&full_bar[s], C::STAGE_BYTES);
          const int k0 = kb * BK;
          if (MODE == MODE_FWD) {
            tma_load_2d(a_dst, &tmA, &full_bar[s], k0, t.row0);
            if (BMN) {
#pragma unroll
              for (int a = 0; a < BN / 64; ++a)
                tma_load_3d(b_dst + a * (BK * 128), &tmB, &full_bar[s], t.n0 + a * 64, k0, t.e);
            } else {
              tma_load_3d(b_dst, &tmB, &full_bar[s], k0, t.n0, t.e);
            }
          } else {
#pragma unroll
            for (int a = 0; a < BM / 64; ++a) tma_load_2d(a_dst + a * (BK * 128), &tmA, &full_bar[s], t.row0 + a * 64, k0);
#pragma unroll
            for (int a = 0; a < BN / 64; ++a) tma_load_2d(b_dst + a * (BK * 128), &tmB, &full_bar[s], t.n0 + a * 64, k0);
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, A_MN, BMN);
      int it = 0, tcount = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const Tile t = decode_tile<MODE>(tile, offs, E, N, K);
        if (t.kb1 <= t.kb0) continue;  // empty expert: nothing to accumulate (epilogue skips it too)
        const int buf = tcount & 1;
        const uint32_t acc_ph = (tcount >> 1) & 1;
        if (!mbar_wait(&tmem_empty[buf], acc_ph ^ 1, abort_flag, status, MT_ERR_TIMEOUT_TMEM_EMPTY)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + buf * BN;
        for (int kb = t.kb0; kb < t.kb1; ++kb, ++it) {
          const int s = it % C::STAGES;
          const uint32_t ph = (it / C::STAGES) & 1;
          if (!mbar_wait(&full_bar[s], ph, abort_flag, status, MT_ERR_TIMEOUT_FULL)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(smem + s * C::STAGE_BYTES);
          const uint32_t b_addr = a_addr + C::A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t da = A_MN ? make_smem_desc_sw128(a_addr + k * (UMMA_K * 128), BK * 128, 1024)
                                     : make_smem_desc_sw128(a_addr + k * (UMMA_K * 2), 16, 1024);
            const uint64_t db = BMN ? make_smem_desc_sw128(b_addr + k * (UMMA_K * 128), BK * 128, 1024)
                                    : make_smem_desc_sw128(b_addr + k * (UMMA_K * 2), 16, 1024);
            tc_mma_f16(d_tmem, da, db, idesc, (kb > t.kb0 || k != 0) ? 1u : 0u);
          }
          tc_commit(&empty_bar[s]);
        }
        if (ok) tc_commit(&tmem_full[buf]);
        ++tcount;
      }
    }
  } else {
    const int q = warp & 3;
    constexpr int COLS = OUT_F32 ? 32 : 64;
    uint8_t* stage0 = epi_base + (warp - 2) * 2 * kEpiStageBytes;
    int tcount = 0, nstores = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      const Tile t = decode_tile<MODE>(tile, offs, E, N, K);
      if (t.kb1 <= t.kb0) continue;
      const int buf = tcount & 1;
      const uint32_t acc_ph = (tcount >> 1) & 1;
      if (!mbar_wait_warp(&tmem_full[buf], acc_ph, abort_flag, status, MT_ERR_TIMEOUT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after_sync();
      const int row0 = t.row0 + q * 32;
      const int row_limit = (MODE == MODE_FWD) ? offs[E] : K;
      const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * BN;
      for (int c = 0; c < BN / COLS; ++c) {
        const int col0 = t.n0 + c * COLS;
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
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          if (row0 < row_limit) {
            if (MODE == MODE_FWD) {
              tma_store_2d(&tmC, sbuf, col0, row0);
            } else if (accumulate) {
              asm volatile(
                  "cp.reduce.async.bulk.tensor.3d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4}], [%1];"
                  ::"l"(reinterpret_cast<uint64_t>(&tmC)), "r"(smem_u32(sbuf)), "r"(col0), "r"(row0), "r"(t.e)
                  : "memory");
            } else {
              tma_store_3d(&tmC, sbuf, col0, row0, t.e);
            }
          }
          tma_commit_group();
        }
        ++nstores;
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[buf]);
      ++tcount;
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

template <typename Kern>
void configure(Kern k) {
  MT_CUDA_CHECK(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, GCfg::SMEM_BYTES));
}

}  // namespace

void set_grouped_variant(int v) { g_variant = (v == 1 || v == 2) ? v : 0; }

void grouped_gemm_bf16(const void* X, const void* W, void* Y, const int* offsets, int E, int M_cap, int N, int K,
                       bool w_mn_major, int* status, int num_sms, cudaStream_t stream) {
  if (M_cap <= 0 || E <= 0) return;
  if (use_pair_kernels() && N > 128 && E <= 256)
    return grouped_gemm_bf16_pair(X, W, Y, offsets, E, M_cap, N, K, w_mn_major, status, num_sms, stream);
  if (E > kMaxExperts) throw std::runtime_error("grouped_gemm_bf16: too many experts");
  const auto bf = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const auto sw = CU_TENSOR_MAP_SWIZZLE_128B;
  CUtensorMap tA = make_tmap_2d(X, bf, 2, M_cap, K, K, BM, BK, sw);
  // W [E, K, N] read MN-major: inner N, rows K ;  W [E, N, K] read K-major: inner K, rows N
  CUtensorMap tB = w_mn_major ? make_tmap_3d(W, bf, 2, E, K, N, (uint64_t)K * N, N, 1, BK, 64, sw)
                              : make_tmap_3d(W, bf, 2, E, N, K, (uint64_t)N * K, K, 1, BN, BK, sw);
  CUtensorMap tC = make_tmap_2d(Y, bf, 2, M_cap, N, N, 32, 64, sw);
  static bool configured = false;
  if (!configured) {
    configure(grouped_gemm_kernel<MODE_FWD, true, false>);
    configure(grouped_gemm_kernel<MODE_FWD, false, false>);
    configured = true;
  }
  if (w_mn_major)
    grouped_gemm_kernel<MODE_FWD, true, false><<<num_sms, kThreads, GCfg::SMEM_BYTES, stream>>>(tA, tB, tC, offsets, E, N, K, 0, status);
  else
    grouped_gemm_kernel<MODE_FWD, false, false><<<num_sms, kThreads, GCfg::SMEM_BYTES, stream>>>(tA, tB, tC, offsets, E, N, K, 0, status);
  MT_CUDA_CHECK(cudaGetLastError());
}

void grouped_wgrad_bf16(const void* X, const void* G, void* dW, const int* offsets, int E, int M_cap, int N, int K,
                        bool out_f32, bool accumulate, int* status, int num_sms, cudaStream_t stream) {
  if (M_cap <= 0 || E <= 0) return;
  if (use_pair_kernels() && N > 128 && K > 128 && E <= 256)
    return grouped_wgrad_bf16_pair(X, G, dW, offsets, E, M_cap, N, K, out_f32, accumulate, status, num_sms, stream);
  if (E > kMaxExperts) throw std::runtime_error("grouped_wgrad_bf16: too many experts");
  const auto bf = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const auto sw = CU_TENSOR_MAP_SWIZZLE_128B;
  CUtensorMap tA = make_tmap_2d(X, bf, 2, M_cap, K, K, BK, 64, sw);
  CUtensorMap tB = make_tmap_2d(G, bf, 2, M_cap, N, N, BK, 64, sw);
  CUtensorMap tC = out_f32 ? make_tmap_3d(dW, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, E, K, N, (uint64_t)K * N, N, 1, 32, 32, sw)
                           : make_tmap_3d(dW, bf, 2, E, K, N, (uint64_t)K * N, N, 1, 32, 64, sw);
  static bool configured = false;
  if (!configured) {
    configure(grouped_gemm_kernel<MODE_WGRAD, true, true>);
    configure(grouped_gemm_kernel<MODE_WGRAD, true, false>);
    configured = true;
  }
  const int tiles = E * ((K + BM - 1) / BM) * ((N + BN - 1) / BN);
  const int grid = tiles < num_sms ? tiles : num_sms;
  if (out_f32)
    grouped_gemm_kernel<MODE_WGRAD, true, true><<<grid, kThreads, GCfg::SMEM_BYTES, stream>>>(tA, tB, tC, offsets, E, N, K, accumulate ? 1 : 0, status);
  else
    grouped_gemm_kernel<MODE_WGRAD, true, false><<<grid, kThreads, GCfg::SMEM_BYTES, stream>>>(tA, tB, tC, offsets, E, N, K, accumulate ? 1 : 0, status);
  MT_CUDA_CHECK(cudaGetLastError());
}

}  // namespace mt
