// Tensor-parallel GEMMs fused with their collectives over NVLink peer memory (sm_100a, bf16, fp32 accumulate).
//
// MODE_AG  all-gather -> GEMM.  C[T, N] = G[T, K] * op(B), where G is the concatenation of every rank's token
//          shard [T/t, K].  The shards live in symmetric memory; G is a local buffer this kernel fills itself:
//          a seventh warp in every CTA pulls 8 KB pieces of the shards (peers' and its own) with bulk TMA copies
//          (peer global -> shared -> local global, two in flight per CTA) and counts finished pieces per
//          128-row block; the TMA producer warp of the GEMM waits (bounded) for a row block's count before it
//          loads A tiles from it.  Tiles are visited starting with this rank's own rows, so the tensor cores
//          work on local data while remote rows are still crossing NVLink.  G stays behind for the caller
//          (further projections of the same input, weight gradients).
// MODE_RS  GEMM -> reduce-scatter.  Every rank computes partial sums for all T rows; the epilogue stores each
//          output tile straight into the staging slot [source rank] of the rank that owns those rows (TMA store
//          to peer memory), so when the kernel ends the partial tiles are already scattered; a small local kernel
//          (tp_reduce_slots) adds the t slots.
// MODE_AGB all-gather of a sharded *weight* -> GEMM (fully-sharded data parallelism).  C[T, N] = A[T, K] * W[K, N] with
//          W sharded over ranks by rows of K.  The gather warps assemble the full W in a local buffer exactly as
//          above; the producer waits per 64-row k-block of W and walks the k-blocks starting with this rank's own
//          shard, so the main loop starts at once and the remote rows arrive underneath it.
// No multicast loads anywhere; remote traffic is bulk / tensor TMA without multicast and ordinary stores.
#include "../common/ptx.cuh"
#include "../common/tmap.h"
#include "../api.h"

namespace mt {
namespace {

constexpr int BM = 128, BN = 256, BK = 64, UMMA_K = 16;
constexpr int kEpiWarps = 4;
constexpr int kThreads = 32 * (3 + kEpiWarps);  // TMA, MMA, 4 epilogue, copy
constexpr int kEpiStageBytes = 4096;
constexpr int kPieceBytes = 8192;  // granularity of the readiness counters
enum { MODE_AG = 0, MODE_RS = 1, MODE_AGB = 2 };

// Shared-memory split per mode: the token gather moves (t-1)/t of the activations and gets a deep copy ring at the
// price of one pipeline stage; the weight gather is small next to its GEMM and keeps four stages; the scattering
// GEMM has no ring at all.
template <int MODE>
struct TCfg {
  static constexpr int kStages = MODE == MODE_AG ? 3 : 4;
  static constexpr int kEpiBufs = MODE == MODE_RS ? 2 : 1;   // staging buffers per epilogue warp
  static constexpr int kCopyBytes = MODE == MODE_AG ? 16384 : 8192;  // bytes per bulk copy (multiple of the piece)
  static constexpr int kCopySlots = MODE == MODE_AG ? 4 : (MODE == MODE_AGB ? 2 : 0);
  static constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int EPI_BYTES = kEpiWarps * kEpiBufs * kEpiStageBytes;
  static constexpr int COPY_BYTES = kCopySlots * kCopyBytes;
  static constexpr int OFF_EPI = kStages * STAGE_BYTES;
  static constexpr int OFF_COPY = OFF_EPI + EPI_BYTES;
  static constexpr int OFF_BAR = OFF_COPY + COPY_BYTES;
  static constexpr int SMEM_BYTES = OFF_BAR + 256;
  static constexpr int TMEM_COLS = 2 * BN;
  static_assert(SMEM_BYTES <= 232448, "shared memory budget");
};

struct CMaps {
  CUtensorMap m[kMaxPeers];
};

struct TpArgs {
  int M, N, K;
  int rank, world;
  int rows_per_rank;      // T / t (multiple of 128)
  // MODE_AG
  const void* shard[kMaxPeers];  // every rank's shard of the gathered operand (symmetric memory)
  void* gathered;                // local buffer for the whole gathered operand
  int* ready;                    // local counters, one per block of the gathered operand: 8 KB pieces landed
  int ready_target;              // value a block's counter has once this call's pieces are in
  int64_t rank_bytes;            // bytes of one rank's shard
  int64_t block_bytes;           // bytes per readiness block (128 token rows of A, or 64 k-rows of W)
  int* status;
};

__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_gpu_add(int* p, int v) {
  asm volatile("red.release.gpu.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(smem_dst)),
               "l"(reinterpret_cast<uint64_t>(gsrc)), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void bulk_s2g(void* gdst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(reinterpret_cast<uint64_t>(gdst)),
               "r"(smem_u32(smem_src)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }

// Tile order: groups of 8 column tiles, rows fastest inside a group, rows rotated so that `row_rot` comes first.
__device__ __forceinline__ void tile_coord(int tile, int num_m, int num_n, int row_rot, int& m_idx, int& n_idx) {
  const int per_group = 8 * num_m;
  const int group = tile / per_group;
  const int first_n = group * 8;
  const int gsize = min(8, num_n - first_n);
  const int local = tile - group * per_group;
  m_idx = (local / gsize + row_rot) % num_m;
  n_idx = first_n + local % gsize;
}

template <int MODE, bool B_MN>
__global__ void __launch_bounds__(kThreads, 1)
tp_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const __grid_constant__ CMaps tmC, const TpArgs a) {
  using C = TCfg<MODE>;
  constexpr int kStages = C::kStages;
  constexpr int kEpiBufs = C::kEpiBufs;
  constexpr int kCopySlots = C::kCopySlots;
  constexpr int kCopyBytes = C::kCopyBytes;
  extern __shared__ __align__(1024) uint8_t smem[];
  if ((smem_u32(smem) & 1023u) != 0) {
    if (threadIdx.x == 0 && a.status) atomicCAS(a.status, 0, MT_ERR_BAD_ARGS);
    return;
  }
  uint8_t* epi_base = smem + C::OFF_EPI;
  uint8_t* copy_base = smem + C::OFF_COPY;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::OFF_BAR);
  uint64_t* full_bar = bars;                 // [kStages]
  uint64_t* empty_bar = bars + kStages;      // [kStages]
  uint64_t* tmem_full = bars + 2 * kStages;  // [2]
  uint64_t* tmem_empty = tmem_full + 2;      // [2]
  uint64_t* copy_bar = tmem_empty + 2;       // [kCopySlots]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(copy_bar + kCopySlots);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_m = (a.M + BM - 1) / BM;
  const int num_n = (a.N + BN - 1) / BN;
  const int num_tiles = num_m * num_n;
  const int num_kb = (a.K + BK - 1) / BK;
  const int blocks_per_rank = a.rows_per_rank / BM;
  const int row_rot = MODE == MODE_AGB ? 0 : a.rank * blocks_per_rank;  // this rank's rows first
  const int kb_rot = MODE == MODE_AGB ? a.rank * (num_kb / a.world) : 0;  // this rank's k-blocks first

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tmem_full[b], 1);
      mbar_init(&tmem_empty[b], kEpiWarps);
    }
    for (int s = 0; s < kCopySlots; ++s) mbar_init(&copy_bar[s], 1);
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmB);
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
    // ------------------------------------------------------------ TMA producer of the GEMM
    if (lane == 0) {
      int it = 0;
      bool ok = true;
      bool all_ready = false;  // MODE_AGB: every k-block has been seen complete (after this CTA's first tile)
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int m_idx, n_idx;
        tile_coord(tile, num_m, num_n, row_rot, m_idx, n_idx);
        if (MODE == MODE_AG) {
          // rows of this block must have been gathered (bounded wait on the landed-pieces counter)
          if (ld_acquire_gpu(a.ready + m_idx) < a.ready_target) {
            const long long t0 = clock64();
            while (ld_acquire_gpu(a.ready + m_idx) < a.ready_target) {
              if (*abort_flag || clock64() - t0 > kMaxWaitCycles) {
                *abort_flag = 1;
                if (a.status) atomicCAS(a.status, 0, MT_ERR_TIMEOUT_FLAG);
                ok = false;
                break;
              }
            }
            if (!ok) break;
          }
          fence_proxy_async_all();
        }
        for (int kbi = 0; kbi < num_kb; ++kbi, ++it) {
          const int kb = (kbi + kb_rot) % num_kb;
          if (MODE == MODE_AGB && !all_ready) {  // this k-block of the weight must have been gathered
            if (ld_acquire_gpu(a.ready + kb) < a.ready_target) {
              const long long t0 = clock64();
              while (ld_acquire_gpu(a.ready + kb) < a.ready_target) {
                if (*abort_flag || clock64() - t0 > kMaxWaitCycles) {
                  *abort_flag = 1;
                  if (a.status) atomicCAS(a.status, 0, MT_ERR_TIMEOUT_FLAG);
                  ok = false;
                  break;
                }
              }
              if (!ok) break;
            }
            fence_proxy_async_all();
          }
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1;
          if (!mbar_wait(&empty_bar[s], ph ^ 1, abort_flag, a.status, MT_ERR_TIMEOUT_EMPTY)) { ok = false; break; }
          uint8_t* a_dst = smem + s * C::STAGE_BYTES;
          uint8_t* b_dst = a_dst + C::A_BYTES;
          mbar_expect_tx(&full_bar[s], C::STAGE_BYTES);
          tma_load_2d(a_dst, &tmA, &full_bar[s], kb * BK, m_idx * BM);
          if (B_MN) {
#pragma unroll
            for (int x = 0; x < BN / 64; ++x)
              tma_load_2d(b_dst + x * (BK * 128), &tmB, &full_bar[s], n_idx * BN + x * 64, kb * BK);
          } else {
            tma_load_2d(b_dst, &tmB, &full_bar[s], kb * BK, n_idx * BN);
          }
        }
        all_ready = true;
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, false, B_MN);
      int it = 0, tcount = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++tcount) {
        const int buf = tcount & 1;
        if (!mbar_wait(&tmem_empty[buf], ((tcount >> 1) & 1) ^ 1, abort_flag, a.status, MT_ERR_TIMEOUT_TMEM_EMPTY)) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + buf * BN;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {  // kb counts loop steps here; the producer chose the k order
          const int s = it % kStages;
          if (!mbar_wait(&full_bar[s], (it / kStages) & 1, abort_flag, a.status, MT_ERR_TIMEOUT_FULL)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(smem + s * C::STAGE_BYTES);
          const uint32_t b_addr = a_addr + C::A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t da = make_smem_desc_sw128(a_addr + k * (UMMA_K * 2), 16, 1024);
            const uint64_t db = B_MN ? make_smem_desc_sw128(b_addr + k * (UMMA_K * 128), BK * 128, 1024)
                                     : make_smem_desc_sw128(b_addr + k * (UMMA_K * 2), 16, 1024);
            tc_mma_f16(d_tmem, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          tc_commit(&empty_bar[s]);
        }
        if (ok) tc_commit(&tmem_full[buf]);
      }
    }
  } else if (warp < 2 + kEpiWarps) {
    // ------------------------------------------------------------ epilogue (bf16 out)
    const int q = warp & 3;
    uint8_t* stage0 = epi_base + (warp - 2) * kEpiBufs * kEpiStageBytes;
    int tcount = 0, nstores = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++tcount) {
      int m_idx, n_idx;
      tile_coord(tile, num_m, num_n, row_rot, m_idx, n_idx);
      const int buf = tcount & 1;
      if (!mbar_wait_warp(&tmem_full[buf], (tcount >> 1) & 1, abort_flag, a.status, MT_ERR_TIMEOUT_TMEM_FULL)) break;
      tc_fence_after_sync();
      int row0 = m_idx * BM + q * 32;
      const CUtensorMap* cmap = &tmC.m[0];
      if (MODE == MODE_RS) {  // rows belong to rank `owner`: store into its staging slot of this source rank
        const int owner = (m_idx * BM) / a.rows_per_rank;
        cmap = &tmC.m[owner];
        row0 -= owner * a.rows_per_rank;
      }
      const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * BN;
      for (int c = 0; c < BN / 64; ++c) {
        const int col0 = n_idx * BN + c * 64;
        if (col0 >= a.N) break;
        uint8_t* sbuf = stage0 + (nstores % kEpiBufs) * kEpiStageBytes;
        if (lane == 0) tma_wait_group_read<kEpiBufs - 1>();
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
          if (m_idx * BM + q * 32 < a.M) tma_store_2d(cmap, sbuf, col0, row0);
          tma_commit_group();
        }
        ++nstores;
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[buf]);
    }
    if (lane == 0) tma_wait_group<0>();
  } else {
    // ------------------------------------------------------------ gather warp: bulk copies of the shards
    if constexpr (MODE == MODE_AG || MODE == MODE_AGB) {
      if (lane == 0) {
        constexpr int kUnitPieces = kCopyBytes / kPieceBytes;
        const int64_t rank_bytes = a.rank_bytes;
        const int64_t units_per_rank = rank_bytes / kCopyBytes;
        const int64_t total = units_per_rank * a.world;
        const int64_t block_bytes = a.block_bytes;
        int64_t mine[kCopySlots];  // copy unit held by each slot
        auto unit_of = [&](int n) -> int64_t {  // n-th unit of this CTA, own rank's region first
          const int64_t i = static_cast<int64_t>(blockIdx.x) + static_cast<int64_t>(n) * gridDim.x;
          return (i + static_cast<int64_t>(a.rank) * units_per_rank) % total;
        };
        auto offset_of = [&](int64_t u) -> int64_t {
          return (u / units_per_rank) * rank_bytes + (u % units_per_rank) * kCopyBytes;
        };
        auto signal = [&](int64_t u) {
          red_release_gpu_add(a.ready + static_cast<int>(offset_of(u) / block_bytes), kUnitPieces);
        };
        const int n_mine = static_cast<int>((total - blockIdx.x + gridDim.x - 1) / gridDim.x);
        int64_t pending_signal = -1;
        bool ok = true;
        for (int n = 0; n < n_mine + (kCopySlots - 1) && ok; ++n) {
          if (n < n_mine) {
            const int s = n % kCopySlots;
            // slot s was last used by unit n - kCopySlots, whose store was issued in the previous iteration
            tma_wait_group_read<0>();
            const int64_t u = unit_of(n);
            mine[s] = u;
            const uint8_t* src =
                static_cast<const uint8_t*>(a.shard[u / units_per_rank]) + (u % units_per_rank) * kCopyBytes;
            mbar_expect_tx(&copy_bar[s], kCopyBytes);
            bulk_g2s(copy_base + s * kCopyBytes, src, kCopyBytes, &copy_bar[s]);
          }
          const int d = n - (kCopySlots - 1);  // unit whose data should have arrived by now
          if (d >= 0 && d < n_mine) {
            const int s = d % kCopySlots;
            if (!mbar_wait(&copy_bar[s], (d / kCopySlots) & 1, abort_flag, a.status, MT_ERR_TIMEOUT_FULL)) {
              ok = false;
              break;
            }
            const int64_t u = mine[s];
            bulk_s2g(static_cast<uint8_t*>(a.gathered) + offset_of(u), copy_base + s * kCopyBytes, kCopyBytes);
            tma_commit_group();
            // the store issued one step earlier has completed once at most one group is pending
            if (pending_signal >= 0) {
              tma_wait_group<1>();
              fence_proxy_async_all();
              signal(pending_signal);
            }
            pending_signal = u;
          }
        }
        tma_wait_group<0>();
        if (ok && pending_signal >= 0) {
          fence_proxy_async_all();
          signal(pending_signal);
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    __syncwarp();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

// y[r, :] = sum over slots of staging[slot][r, :]   (bf16 in, fp32 add, bf16 out)
__global__ void tp_reduce_slots_kernel(const __nv_bfloat16* __restrict__ staging, __nv_bfloat16* __restrict__ y,
                                       int slots, int64_t slot_elems) {
  const int64_t nvec = slot_elems >> 3;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (int64_t)gridDim.x * blockDim.x) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int s = 0; s < slots; ++s) {
      const uint4 v = reinterpret_cast<const uint4*>(staging + s * slot_elems)[i];
      const __nv_bfloat16* h = reinterpret_cast<const __nv_bfloat16*>(&v);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += __bfloat162float(h[j]);
    }
    uint4 o;
    o.x = pack_bf16x2(acc[0], acc[1]);
    o.y = pack_bf16x2(acc[2], acc[3]);
    o.z = pack_bf16x2(acc[4], acc[5]);
    o.w = pack_bf16x2(acc[6], acc[7]);
    reinterpret_cast<uint4*>(y)[i] = o;
  }
}

template <int MODE, bool B_MN>
void launch(const CUtensorMap& tA, const CUtensorMap& tB, const CMaps& tC, const TpArgs& a, int num_sms,
            cudaStream_t stream) {
  auto kern = tp_gemm_kernel<MODE, B_MN>;
  using Cf = TCfg<MODE>;
  static bool configured = false;
  if (!configured) {
    MT_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cf::SMEM_BYTES));
    configured = true;
  }
  const int tiles = ((a.M + BM - 1) / BM) * ((a.N + BN - 1) / BN);
  const int grid = tiles < num_sms ? tiles : num_sms;
  kern<<<grid, kThreads, Cf::SMEM_BYTES, stream>>>(tA, tB, tC, a);
  MT_CUDA_CHECK(cudaGetLastError());
}

}  // namespace

void tp_gemm_ag(const PeerPtrs& shards, void* gathered, const void* B, void* Cout, int T, int N, int K, int rank,
                int world, bool b_mn_major, int* ready, int ready_target, int* status, int num_sms,
                cudaStream_t stream) {
  const int rows_per_rank = T / world;
  if (T % (world * BM) != 0) throw std::runtime_error("tp_gemm_ag: tokens per rank must be a multiple of 128");
  if (K % 64 != 0) throw std::runtime_error("tp_gemm_ag: K must be a multiple of 64");
  const auto bf = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const auto sw = CU_TENSOR_MAP_SWIZZLE_128B;
  CUtensorMap tA = make_tmap_2d(gathered, bf, 2, T, K, K, BM, BK, sw);
  CUtensorMap tB = b_mn_major ? make_tmap_2d(B, bf, 2, K, N, N, BK, 64, sw) : make_tmap_2d(B, bf, 2, N, K, K, BN, BK, sw);
  CMaps tC{};
  tC.m[0] = make_tmap_2d(Cout, bf, 2, T, N, N, 32, 64, sw);
  TpArgs a{};
  a.M = T; a.N = N; a.K = K; a.rank = rank; a.world = world; a.rows_per_rank = rows_per_rank;
  for (int i = 0; i < world; ++i) a.shard[i] = shards.p[i];
  a.gathered = gathered; a.ready = ready; a.ready_target = ready_target; a.status = status;
  a.rank_bytes = static_cast<int64_t>(rows_per_rank) * K * 2;
  a.block_bytes = static_cast<int64_t>(BM) * K * 2;
  if (b_mn_major) launch<MODE_AG, true>(tA, tB, tC, a, num_sms, stream);
  else launch<MODE_AG, false>(tA, tB, tC, a, num_sms, stream);
}

void tp_gemm_rs(const void* A, const void* B, const PeerPtrs& staging_slots, int T, int N, int K, int rank, int world,
                bool b_mn_major, int* status, int num_sms, cudaStream_t stream) {
  const int rows_per_rank = T / world;
  if (T % (world * BM) != 0) throw std::runtime_error("tp_gemm_rs: tokens per rank must be a multiple of 128");
  const auto bf = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const auto sw = CU_TENSOR_MAP_SWIZZLE_128B;
  CUtensorMap tA = make_tmap_2d(A, bf, 2, T, K, K, BM, BK, sw);
  CUtensorMap tB = b_mn_major ? make_tmap_2d(B, bf, 2, K, N, N, BK, 64, sw) : make_tmap_2d(B, bf, 2, N, K, K, BN, BK, sw);
  CMaps tC{};
  for (int i = 0; i < world; ++i)  // staging_slots.p[i]: rank i's slot reserved for this source rank, [T/t, N]
    tC.m[i] = make_tmap_2d(staging_slots.p[i], bf, 2, rows_per_rank, N, N, 32, 64, sw);
  TpArgs a{};
  a.M = T; a.N = N; a.K = K; a.rank = rank; a.world = world; a.rows_per_rank = rows_per_rank; a.status = status;
  if (b_mn_major) launch<MODE_RS, true>(tA, tB, tC, a, num_sms, stream);
  else launch<MODE_RS, false>(tA, tB, tC, a, num_sms, stream);
}

void fsdp_gemm_agw(const void* A, const PeerPtrs& w_shards, void* w_full, void* Cout, int T, int N, int K, int rank,
                   int world, int* ready, int* status, int num_sms, cudaStream_t stream) {
  if (K % (world * BK) != 0) throw std::runtime_error("fsdp_gemm_agw: K must be a multiple of 64 * world");
  if ((static_cast<int64_t>(BK) * N * 2) % kPieceBytes != 0 || (static_cast<int64_t>(K / world) * N * 2) % kPieceBytes != 0)
    throw std::runtime_error("fsdp_gemm_agw: N must be a multiple of 128");
  const auto bf = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const auto sw = CU_TENSOR_MAP_SWIZZLE_128B;
  CUtensorMap tA = make_tmap_2d(A, bf, 2, T, K, K, BM, BK, sw);
  CUtensorMap tB = make_tmap_2d(w_full, bf, 2, K, N, N, BK, 64, sw);
  CMaps tC{};
  tC.m[0] = make_tmap_2d(Cout, bf, 2, T, N, N, 32, 64, sw);
  TpArgs a{};
  a.M = T; a.N = N; a.K = K; a.rank = rank; a.world = world; a.rows_per_rank = BM;  // unused by this mode
  for (int i = 0; i < world; ++i) a.shard[i] = w_shards.p[i];
  a.gathered = w_full; a.ready = ready; a.status = status;
  a.rank_bytes = static_cast<int64_t>(K / world) * N * 2;
  a.block_bytes = static_cast<int64_t>(BK) * N * 2;
  a.ready_target = static_cast<int>(a.block_bytes / kPieceBytes);
  launch<MODE_AGB, true>(tA, tB, tC, a, num_sms, stream);
}

void tp_reduce_slots(const void* staging, void* y, int slots, int64_t slot_elems, cudaStream_t stream) {
  if (slot_elems == 0) return;
  int64_t b = (slot_elems / 8 + 255) / 256;
  if (b > 148 * 16) b = 148 * 16;
  tp_reduce_slots_kernel<<<(int)b, 256, 0, stream>>>((const __nv_bfloat16*)staging, (__nv_bfloat16*)y, slots, slot_elems);
}

}  // namespace mt
