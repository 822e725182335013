// Backward of the gated activation fused into the data-gradient GEMM of the down projection, on CTA pairs
// (tcgen05 cta_group::2):
//     dH = dY Wd^T                       dY [T, D] bf16, Wd [I, D] bf16 (as the parameter is stored)
//     dG = dH * U * act'(G)   dU = dH * act(G)          G, U: the halves of the forward's [T, 2I] buffer
// dH never reaches memory: each epilogue warp fetches the G and U boxes that match its 32 x 64 accumulator chunk by
// TMA (one chunk ahead, into the staging buffers that afterwards carry dG and dU out), combines them with the
// accumulator in registers and stores dG | dU into the halves of a [T, 2I] buffer - the operand of the gate / up
// data- and weight-gradient GEMMs.  The stand-alone backward activation kernel and the write + read of dH are gone
// (mintext/modules/linear.py:218-225 for the layer).  Main loop, barriers, bounded waits and the absence of multicast
// loads are those of dense_bf16_2cta.cu; five ring stages leave room for four staging boxes per epilogue warp.
#include "../common/ptx.cuh"
#include "../common/tmap.h"
#include "../common/pair.cuh"
#include "../api.h"

namespace mt {
namespace {

constexpr int BM = 128;        // rows per CTA (256 per pair)
constexpr int BN = 256;        // columns (of I) per pair tile; each CTA stages BN/2 rows of Wd
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int kEpiWarps = 4;
constexpr int kThreads = 32 * (2 + kEpiWarps);
constexpr int kBoxBytes = 4096;  // 32 rows x 64 bf16
constexpr int kStages = 5;
constexpr int kChunks = BN / 64;

struct BCfg {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = (BN / 2) * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int EPI_BYTES = kEpiWarps * 4 * kBoxBytes;  // per warp: two sets of (G -> dG, U -> dU) boxes
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

// value and derivative of the activation (codes of the stand-alone kernels: 0 silu, 1 gelu-tanh, 2 gelu-erf, 3 relu)
template <int ACT>
__device__ __forceinline__ void act_and_grad(float x, float& f, float& df) {
  if (ACT == 0) {
    const float s = 1.f / (1.f + __expf(-x));
    f = x * s;
    df = s * (1.f + x * (1.f - s));
  } else if (ACT == 1) {
    const float k0 = 0.7978845608028654f, k1 = 0.044715f;
    const float t = tanhf(k0 * (x + k1 * x * x * x));
    f = 0.5f * x * (1.f + t);
    df = 0.5f * (1.f + t) + 0.5f * x * (1.f - t * t) * k0 * (1.f + 3.f * k1 * x * x);
  } else if (ACT == 2) {
    const float e = erff(x * 0.7071067811865476f);
    f = 0.5f * x * (1.f + e);
    df = 0.5f * (1.f + e) + x * 0.3989422804014327f * __expf(-0.5f * x * x);
  } else {
    f = x > 0.f ? x : 0.f;
    df = x > 0.f ? 1.f : 0.f;
  }
}

__device__ __forceinline__ float bf16_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }

template <int ACT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
gemm_gated_bwd_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                           const __grid_constant__ CUtensorMap tmGU, const __grid_constant__ CUtensorMap tmDGU, int T,
                           int I, int K, int* status) {
  using C = BCfg;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* epi_base = smem + C::OFF_EPI;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::OFF_BAR);
  uint64_t* full_bar = bars;                   // leader only
  uint64_t* empty_bar = bars + kStages;        // per CTA
  uint64_t* tmem_full = bars + 2 * kStages;    // per CTA
  uint64_t* tmem_empty = tmem_full + 2;        // leader only (8 arrivals)
  uint64_t* box_bar = tmem_empty + 2;          // [kEpiWarps][2] per epilogue warp and staging set: G / U boxes landed
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(box_bar + 2 * kEpiWarps);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  const int num_m = (T + 2 * BM - 1) / (2 * BM);
  const int num_n = I / BN;
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
    for (int w = 0; w < 2 * kEpiWarps; ++w) mbar_init(&box_bar[w], 1);
    *abort_flag = aligned ? 0 : 1;
    if (!aligned && status) atomicCAS(status, 0, MT_ERR_BAD_ARGS);
    fence_barrier_init();
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmB);
    prefetch_tmap(&tmGU);
    prefetch_tmap(&tmDGU);
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
      int it = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        int m_idx, n_idx;
        tile_coord(tile, num_m, num_n, m_idx, n_idx);
        const int row0 = m_idx * (2 * BM) + rank * BM;       // this CTA's rows of dY
        const int col0 = n_idx * BN + rank * (BN / 2);       // this CTA's rows of Wd (= columns of dH)
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % kStages;
          if (!mbar_wait(&empty_bar[s], ((it / kStages) & 1) ^ 1, abort_flag, status, MT_ERR_TIMEOUT_EMPTY)) {
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
    // ------------------------------------------------------------ MMA issuer (leader CTA only)
    if (lane == 0 && leader && aligned) {
      constexpr uint32_t idesc = make_idesc_bf16(2 * BM, BN, false, false);
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
          const uint64_t da = make_smem_desc_sw128(a_addr, 16, 1024);
          const uint64_t db = make_smem_desc_sw128(a_addr + C::A_BYTES, 16, 1024);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            tc_mma_f16_pair(d_tmem, da + k * ((UMMA_K * 2) >> 4), db + k * ((UMMA_K * 2) >> 4), idesc, (kb | k) != 0 ? 1u : 0u);
          tc_commit_pair(&empty_bar[s]);
        }
        if (ok) tc_commit_pair(&tmem_full[buf]);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (both CTAs, own 128 rows)
    // Work items = (tile, 64-column chunk).  Item n uses staging set n & 1 of this warp: its G and U boxes arrive by
    // TMA (issued one item ahead), are read into registers, and the same two boxes then carry dG and dU out.
    const int q = warp & 3;
    const int ew = warp - 2;
    uint8_t* wbase = epi_base + ew * 4 * kBoxBytes;
    uint64_t* my_bar = &box_bar[2 * ew];  // one barrier per staging set: a set's next fetch may start before the other's lands
    auto item_coords = [&](int tile, int c, int& row, int& col) {
      int m_idx, n_idx;
      tile_coord(tile, num_m, num_n, m_idx, n_idx);
      row = m_idx * (2 * BM) + rank * BM + q * 32;
      col = n_idx * BN + c * 64;
    };
    auto fetch = [&](int n, int tile, int c) {  // lane 0 only
      int row, col;
      item_coords(tile, c, row, col);
      uint8_t* set = wbase + (n & 1) * 2 * kBoxBytes;
      tma_wait_group_read<0>();  // the stores that last used this set have read it
      mbar_expect_tx(&my_bar[n & 1], 2 * kBoxBytes);
      tma_load_2d(set, &tmGU, &my_bar[n & 1], col, row);
      tma_load_2d(set + kBoxBytes, &tmGU, &my_bar[n & 1], I + col, row);
    };
    int n = 0, tcount = 0;
    bool ok = aligned;
    if (ok && pair < num_tiles && lane == 0) fetch(0, pair, 0);
    for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, ++tcount) {
      const int buf = tcount & 1;
      if (!mbar_wait_warp(&tmem_full[buf], (tcount >> 1) & 1, abort_flag, status, MT_ERR_TIMEOUT_TMEM_FULL)) break;
      tc_fence_after_sync();
      const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * BN;
#pragma unroll 1
      for (int c = 0; c < kChunks; ++c, ++n) {
        const int next_tile = c + 1 < kChunks ? tile : tile + num_pairs;
        if (lane == 0 && next_tile < num_tiles) fetch(n + 1, next_tile, (c + 1) % kChunks);
        if (!mbar_wait_warp(&my_bar[n & 1], (n >> 1) & 1, abort_flag, status, MT_ERR_TIMEOUT_FULL)) {
          ok = false;
          break;
        }
        int row, col;
        item_coords(tile, c, row, col);
        uint8_t* gbox = wbase + (n & 1) * 2 * kBoxBytes;
        uint8_t* ubox = gbox + kBoxBytes;
        uint8_t* grow = gbox + lane * 128;
        uint8_t* urow = ubox + lane * 128;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(t_lane + c * 64 + h * 32, r);
          tc_wait_ld();
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int off = ((h * 4 + j) ^ (lane & 7)) << 4;
            const uint4 gv = *reinterpret_cast<const uint4*>(grow + off);
            const uint4 uv = *reinterpret_cast<const uint4*>(urow + off);
            const uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w}, uw[4] = {uv.x, uv.y, uv.z, uv.w};
            uint32_t dgw[4], duw[4];
#pragma unroll
            for (int p = 0; p < 4; ++p) {
              float f0, d0, f1, d1;
              act_and_grad<ACT>(bf16_lo(gw[p]), f0, d0);
              act_and_grad<ACT>(bf16_hi(gw[p]), f1, d1);
              const float h0 = __uint_as_float(r[8 * j + 2 * p]), h1 = __uint_as_float(r[8 * j + 2 * p + 1]);
              dgw[p] = pack_bf16x2(h0 * bf16_lo(uw[p]) * d0, h1 * bf16_hi(uw[p]) * d1);
              duw[p] = pack_bf16x2(h0 * f0, h1 * f1);
            }
            *reinterpret_cast<uint4*>(grow + off) = make_uint4(dgw[0], dgw[1], dgw[2], dgw[3]);
            *reinterpret_cast<uint4*>(urow + off) = make_uint4(duw[0], duw[1], duw[2], duw[3]);
          }
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          if (row < T) {
            tma_store_2d(&tmDGU, gbox, col, row);
            tma_store_2d(&tmDGU, ubox, I + col, row);
          }
          tma_commit_group();
        }
      }
      if (!ok) break;
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
void launch_gated_bwd(const CUtensorMap& tA, const CUtensorMap& tB, const CUtensorMap& tGU, const CUtensorMap& tDGU, int T,
                      int I, int K, int* status, int num_sms, cudaStream_t stream) {
  auto kern = gemm_gated_bwd_pair_kernel<ACT>;
  static bool configured = false;
  if (!configured) {
    MT_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, BCfg::SMEM_BYTES));
    configured = true;
  }
  const int tiles = ((T + 2 * BM - 1) / (2 * BM)) * (I / BN);
  const int max_pairs = num_sms / 2;
  const int pairs = tiles < max_pairs ? tiles : max_pairs;
  kern<<<2 * pairs, kThreads, BCfg::SMEM_BYTES, stream>>>(tA, tB, tGU, tDGU, T, I, K, status);
  MT_CUDA_CHECK(cudaGetLastError());
}

}  // namespace

// dY [T, D] (row pitch ldy); Wd [I, D] contiguous; GU, dGU [T, 2I] contiguous bf16.  I % 256 == 0, D % 8 == 0.
void gemm_gated_bwd_pair(const void* dY, const void* Wd, const void* GU, void* dGU, int T, int I, int D, int64_t ldy,
                         int act, int* status, int num_sms, cudaStream_t stream) {
  if (T <= 0 || I <= 0 || D <= 0) return;
  if (I % BN != 0 || D % 8 != 0) throw std::runtime_error("gemm_gated_bwd_pair: I must be a multiple of 256, D of 8");
  const auto bf = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const auto sw = CU_TENSOR_MAP_SWIZZLE_128B;
  CUtensorMap tA = make_tmap_2d(dY, bf, 2, T, D, ldy, BM, BK, sw);
  CUtensorMap tB = make_tmap_2d(Wd, bf, 2, I, D, D, BN / 2, BK, sw);
  CUtensorMap tGU = make_tmap_2d(GU, bf, 2, T, 2 * I, 2 * I, 32, 64, sw);
  CUtensorMap tDGU = make_tmap_2d(dGU, bf, 2, T, 2 * I, 2 * I, 32, 64, sw);
  switch (act) {
    case 0: return launch_gated_bwd<0>(tA, tB, tGU, tDGU, T, I, D, status, num_sms, stream);
    case 1: return launch_gated_bwd<1>(tA, tB, tGU, tDGU, T, I, D, status, num_sms, stream);
    case 2: return launch_gated_bwd<2>(tA, tB, tGU, tDGU, T, I, D, status, num_sms, stream);
    default: return launch_gated_bwd<3>(tA, tB, tGU, tDGU, T, I, D, status, num_sms, stream);
  }
}

}  // namespace mt
