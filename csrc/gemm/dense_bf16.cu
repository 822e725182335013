// Dense bf16 GEMM for sm_100a:  C[M,N] (+)= op(A) * op(B), fp32 accumulation in tensor memory.
//
// Structure (one persistent CTA per SM, 192 threads):
//   warp 0      TMA producer  : streams 128x64 (A) and BNx64 (B) bf16 tiles into a shared-memory ring
//   warp 1      MMA issuer    : one thread issues tcgen05.mma (M=128, N=BN, K=16) on smem descriptors;
//                               tcgen05.commit releases ring slots and publishes finished accumulators
//   warps 2..5  epilogue      : tcgen05.ld the accumulator (double-buffered in TMEM so the next tile's
//                               main loop overlaps), convert, stage in swizzled smem, TMA store / TMA add
// Operand layouts: each of A and B may be "K-major" (contraction dim contiguous: A is [M,K], B is [N,K])
// or "MN-major" (A given as [K,M], B given as [K,N]); this covers forward, dgrad and wgrad of a linear
// layer without any transpose pass.  All ragged edges are handled by TMA zero-fill / clipping.
// Every mbarrier wait is bounded; on expiry the CTA records a code in `status` and unwinds.
#include "../common/ptx.cuh"
#include "../common/tmap.h"
#include "../api.h"
#include <cstdlib>

namespace mt {
namespace {

constexpr int BM = 128;
constexpr int BK = 64;       // 64 bf16 = 128 bytes = one swizzle span
constexpr int UMMA_K = 16;
constexpr int kEpiWarps = 4;
constexpr int kThreads = 32 * (2 + kEpiWarps);
constexpr int kSmemLimit = 232448;  // 227 KB
constexpr int kEpiStageBytes = 4096;  // 32 rows x 128 B per warp per buffer
constexpr int kGroupN = 8;

template <int BN>
struct Cfg {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int EPI_BYTES = kEpiWarps * 2 * kEpiStageBytes;
  static constexpr int BAR_BYTES = 1024;
  static constexpr int STAGES_RAW = (kSmemLimit - 1024 - EPI_BYTES - BAR_BYTES) / STAGE_BYTES;
  static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
  static constexpr int SMEM_BYTES = 1024 + STAGES * STAGE_BYTES + EPI_BYTES + BAR_BYTES;
  static constexpr int TMEM_COLS = 2 * BN;
  static_assert(STAGES >= 2, "need at least a double buffer");
  static_assert(TMEM_COLS <= 512, "TMEM has 512 columns");
};

struct TileCoord {
  int m0, n0;
};

__device__ __forceinline__ TileCoord tile_coord(int tile, int num_m, int num_n, int BN) {
  const int per_group = kGroupN * num_m;
  const int group = tile / per_group;
  const int first_n = group * kGroupN;
  const int gsize = min(kGroupN, num_n - first_n);
  const int local = tile - group * per_group;
  TileCoord t;
  t.m0 = (local / gsize) * BM;
  t.n0 = (first_n + local % gsize) * BN;
  return t;
}

template <int BN, bool A_MN, bool B_MN, bool OUT_F32>
__global__ void __launch_bounds__(kThreads, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmC, int M, int N, int K, int accumulate, int splits,
                 int* status) {
  using C = Cfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* epi_base = smem + C::STAGES * C::STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(epi_base + C::EPI_BYTES);
  uint64_t* full_bar = bars;                    // [STAGES]
  uint64_t* empty_bar = bars + C::STAGES;       // [STAGES]
  uint64_t* tmem_full = bars + 2 * C::STAGES;   // [2]
  uint64_t* tmem_empty = tmem_full + 2;         // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_m = (M + BM - 1) / BM;
  const int num_n = (N + BN - 1) / BN;
  const int num_tiles = num_m * num_n;
  const int num_kb = (K + BK - 1) / BK;
  // split-K (only with the accumulating epilogue): work item w = split * num_tiles + tile covers k-blocks
  // [split * num_kb / splits, (split + 1) * num_kb / splits)
  const int num_items = num_tiles * splits;

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

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int it = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x) {
        const int split = item / num_tiles;
        const TileCoord tc = tile_coord(item - split * num_tiles, num_m, num_n, BN);
        const int kb_lo = static_cast<int>(static_cast<int64_t>(split) * num_kb / splits);
        const int kb_hi = static_cast<int>(static_cast<int64_t>(split + 1) * num_kb / splits);
        for (int kb = kb_lo; kb < kb_hi; ++kb, ++it) {
          const int s = it % C::STAGES;
          const uint32_t ph = (it / C::STAGES) & 1;
          if (!mbar_wait(&empty_bar[s], ph ^ 1, abort_flag, status, MT_ERR_TIMEOUT_EMPTY)) {
            ok = false;
            break;
          }
          uint8_t* a_dst = smem + s * C::STAGE_BYTES;
          uint8_t* b_dst = a_dst + C::A_BYTES;
          mbar_expect_tx(&full_bar[s], C::STAGE_BYTES);
          const int k0 = kb * BK;
          if constexpr (A_MN) {
#pragma unroll
            for (int a = 0; a < BM / 64; ++a) tma_load_2d(a_dst + a * (BK * 128), &tmA, &full_bar[s], tc.m0 + a * 64, k0);
          } else {
            tma_load_2d(a_dst, &tmA, &full_bar[s], k0, tc.m0);
          }
          if constexpr (B_MN) {
#pragma unroll
            for (int a = 0; a < BN / 64; ++a) tma_load_2d(b_dst + a * (BK * 128), &tmB, &full_bar[s], tc.n0 + a * 64, k0);
          } else {
            tma_load_2d(b_dst, &tmB, &full_bar[s], k0, tc.n0);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, A_MN, B_MN);
      int it = 0;
      int tcount = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x, ++tcount) {
        const int split = item / num_tiles;
        const int kb_lo = static_cast<int>(static_cast<int64_t>(split) * num_kb / splits);
        const int kb_hi = static_cast<int>(static_cast<int64_t>(split + 1) * num_kb / splits);
        const int buf = tcount & 1;
        const uint32_t acc_ph = (tcount >> 1) & 1;
        if (!mbar_wait(&tmem_empty[buf], acc_ph ^ 1, abort_flag, status, MT_ERR_TIMEOUT_TMEM_EMPTY)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + buf * BN;
        for (int kb = kb_lo; kb < kb_hi; ++kb, ++it) {
          const int s = it % C::STAGES;
          const uint32_t ph = (it / C::STAGES) & 1;
          if (!mbar_wait(&full_bar[s], ph, abort_flag, status, MT_ERR_TIMEOUT_FULL)) {
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
            tc_mma_f16(d_tmem, da, db, idesc, ((kb - kb_lo) | k) != 0 ? 1u : 0u);
          }
          tc_commit(&empty_bar[s]);  // slot reusable once these MMAs have read it
        }
        if (ok) tc_commit(&tmem_full[buf]);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    constexpr int COLS = OUT_F32 ? 32 : 64;  // columns per 128-byte staging row
    uint8_t* stage0 = epi_base + (warp - 2) * 2 * kEpiStageBytes;
    int tcount = 0;
    int nstores = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x, ++tcount) {
      const TileCoord tc = tile_coord(item % num_tiles, num_m, num_n, BN);
      const int buf = tcount & 1;
      const uint32_t acc_ph = (tcount >> 1) & 1;
      if (!mbar_wait_warp(&tmem_full[buf], acc_ph, abort_flag, status, MT_ERR_TIMEOUT_TMEM_FULL)) {
        ok = false;
        break;
      }
      tc_fence_after_sync();
      const int row0 = tc.m0 + q * 32;
      const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * BN;
      for (int c = 0; c < BN / COLS; ++c) {
        const int col0 = tc.n0 + c * COLS;
        if (col0 >= N) break;
        uint8_t* sbuf = stage0 + (nstores & 1) * kEpiStageBytes;
        // the store issued two boxes ago read this buffer; make sure it is done
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
              const int chunk = h * 4 + j;
              *reinterpret_cast<uint4*>(srow + ((chunk ^ (lane & 7)) << 4)) = v;
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
      // accumulator buffer fully read by this warp
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[buf]);
    }
    if (lane == 0) tma_wait_group<0>();
  }

  // ---------------------------------------------------------------- teardown
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    __syncwarp();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

template <int BN, bool A_MN, bool B_MN, bool OUT_F32>
void launch_variant(const CUtensorMap& tA, const CUtensorMap& tB, const CUtensorMap& tC, int M, int N, int K,
                    bool accumulate, int* status, int num_sms, cudaStream_t stream) {
  using C = Cfg<BN>;
  auto kern = gemm_bf16_kernel<BN, A_MN, B_MN, OUT_F32>;
  static bool configured = false;
  if (!configured) {
    MT_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES));
    configured = true;
  }
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  // Split K when the tiles fill the last wave badly and the epilogue adds into C anyway (weight gradients:
  // few tiles, long K).  Each split pays one more pass of the fp32 tile through the reduce-add epilogue.
  int splits = 1;
  if (OUT_F32 && accumulate) {
    const int num_kb = (K + BK - 1) / BK;
    auto eff = [&](int s) {
      const int items = tiles * s;
      return static_cast<double>(items) / (static_cast<double>((items + num_sms - 1) / num_sms) * num_sms);
    };
    double best = eff(1);
    for (int s = 2; s <= 4; ++s) {
      if (num_kb / s < 16) break;
      if (eff(s) > best + 0.08) {
        best = eff(s);
        splits = s;
      }
    }
  }
  const int items = tiles * splits;
  const int grid = items < num_sms ? items : num_sms;
  kern<<<grid, kThreads, C::SMEM_BYTES, stream>>>(tA, tB, tC, M, N, K, accumulate ? 1 : 0, splits, status);
  MT_CUDA_CHECK(cudaGetLastError());
}

template <int BN>
void launch_bn(bool a_mn, bool b_mn, bool out_f32, const CUtensorMap& tA, const CUtensorMap& tB,
               const CUtensorMap& tC, int M, int N, int K, bool accumulate, int* status, int num_sms,
               cudaStream_t stream) {
#define MT_GEMM_CASE(AM, BMJ, F32)                                                                      \
  if (a_mn == AM && b_mn == BMJ && out_f32 == F32)                                                      \
    return launch_variant<BN, AM, BMJ, F32>(tA, tB, tC, M, N, K, accumulate, status, num_sms, stream);
  MT_GEMM_CASE(false, false, false)
  MT_GEMM_CASE(false, true, false)
  MT_GEMM_CASE(true, false, false)
  MT_GEMM_CASE(true, true, false)
  MT_GEMM_CASE(false, false, true)
  MT_GEMM_CASE(false, true, true)
  MT_GEMM_CASE(true, false, true)
  MT_GEMM_CASE(true, true, true)
#undef MT_GEMM_CASE
}

}  // namespace

// A: K-major -> [M,K] with row pitch lda; MN-major -> [K,M] with row pitch lda.  Same for B with N.
// C: [M,N] row pitch ldc, bf16 or fp32.  accumulate -> C += result (TMA element-wise add).
void gemm_bf16(const void* A, const void* B, void* Cout, int M, int N, int K, int64_t lda, int64_t ldb,
               int64_t ldc, bool a_mn_major, bool b_mn_major, bool out_f32, bool accumulate, int* status,
               int num_sms, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return;
  // Two-SM tiles (256x256 per CTA pair) wherever a whole pair tile is useful; the single-CTA kernel keeps narrow
  // outputs and short row counts.  MT_GEMM_SINGLE_CTA=1 forces the single-CTA kernel (for comparisons).
  static const bool single_only = [] {
    const char* e = std::getenv("MT_GEMM_SINGLE_CTA");
    return e != nullptr && e[0] == '1';
  }();
  if (!single_only && M > 128 && N > 128)
    return gemm_bf16_pair(A, B, Cout, M, N, K, lda, ldb, ldc, a_mn_major, b_mn_major, out_f32, accumulate, status,
                          num_sms, stream);
  const int BN = (N <= 128) ? 128 : 256;
  const auto bf = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const auto sw = CU_TENSOR_MAP_SWIZZLE_128B;
  CUtensorMap tA = a_mn_major ? make_tmap_2d(A, bf, 2, K, M, lda, BK, 64, sw) : make_tmap_2d(A, bf, 2, M, K, lda, BM, BK, sw);
  CUtensorMap tB = b_mn_major ? make_tmap_2d(B, bf, 2, K, N, ldb, BK, 64, sw)
                              : make_tmap_2d(B, bf, 2, N, K, ldb, BN, BK, sw);
  CUtensorMap tC = out_f32 ? make_tmap_2d(Cout, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, M, N, ldc, 32, 32, sw)
                           : make_tmap_2d(Cout, bf, 2, M, N, ldc, 32, 64, sw);
  if (BN == 128) launch_bn<128>(a_mn_major, b_mn_major, out_f32, tA, tB, tC, M, N, K, accumulate, status, num_sms, stream);
  else launch_bn<256>(a_mn_major, b_mn_major, out_f32, tA, tB, tC, M, N, K, accumulate, status, num_sms, stream);
}

}  // namespace mt
