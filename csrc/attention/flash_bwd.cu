// Flash attention backward for sm_100a (bf16, head_dim 64, 128 or 256, the 192/128 multi-head-latent shape,
// grouped-query K/V, causal / sliding window / soft-cap).
//
// One CTA = one (batch, kv head, 128-key block).  It keeps K_j and V_j in shared memory and dK_j, dV_j as fp32
// accumulators in tensor memory while it walks over every query head of the group and every 128-row query
// block that can see the key block.  Per (query head, query block) five tcgen05 MMAs run:
//     S^T  = K_j Q_i^T          dP^T = V_j dO_i^T                      (both M=128 keys, N=128 queries, K=dh)
//     dV  += P^T dO_i           dK  += dS^T Q_i                        (M=128 keys, N=dh, K=128 queries)
//     dQ_i = dS K_j                                                     (M=128 queries, N=dh, K=128 keys)
// The score tiles are produced transposed (keys on TMEM lanes) so that P^T and dS^T, written once to swizzled
// shared memory by the 128 softmax threads (thread = key row), serve as the K-major A operand of dV / dK and,
// read with an MN-major descriptor, as the A operand of dQ; Q_i and dO_i tiles likewise serve as K-major B of
// the first pair and MN-major B of the second pair.  dQ partials leave through a per-warp TMA reduce-add into
// an fp32 accumulator.  A small pre-pass computes delta = rowsum(dO * O) and clears the dQ accumulator; a
// post-pass converts dQ to bf16.
// head_dim 128 does not fit five 128-column accumulators into the 512 columns of tensor memory, so it walks the
// queries in blocks of 64 (S^T, dP^T: N = 64) and produces dQ transposed, dQ_i^T = K_j^T dS^T (M = dh, N = 64
// queries: the same two shared-memory tiles with the operand roles swapped); the drain transposes it back through
// the staging slab of the TMA reduce-add.  The multi-head-latent shape (192-wide queries / keys, 128-wide values)
// uses 32-query steps; its dQ^T needs 192 lanes, so it is produced as two M = 128 groups over head dims 0..127 and
// 64..191 (the second one's upper 64 lanes are the new dims), each 64 columns wide (the upper 32 are never read).
// head_dim 256 also uses 32-query steps and two dQ^T groups (dims 0..127, 128..255), and runs as two launches: one
// that forms P^T and accumulates dV, one that forms dS^T and accumulates dK and dQ (see BwdCfg).
// Roles: eight softmax / epilogue warps (two per 32-key lane quarter of tensor memory, each taking half of the step's
// query columns, so that every scheduler has two of them to overlap latencies; four for the 32-query MLA steps),
// then one TMA producer warp and one MMA issuer warp.  All mbarrier waits are bounded.
#include "../common/ptx.cuh"
#include "../common/tmap.h"
#include <type_traits>
#include "../api.h"
#include <cstdlib>

namespace mt {
namespace {

constexpr int BKV = 128;  // keys per CTA
constexpr float kLog2e = 1.4426950408889634f;

// PASS: 0 = every gradient in one launch; 1 = dV only; 2 = dK and dQ only.  head_dim 256 runs as passes 1 and 2:
// dK and dV alone (256 fp32 columns each) would fill tensor memory, and K, V, Q and dO tiles together leave no room
// for both score staging buffers in shared memory.
template <int DQK, int DV, int PASS = 0>
struct BwdCfg {
  static constexpr bool HAS_DV = PASS != 2;         // P^T staged, dV accumulated
  static constexpr bool HAS_DK = PASS != 1;         // V loaded, dP^T / dS^T formed, dK and dQ accumulated
  static constexpr int BQ = DQK == 64 ? 128 : (DQK == 128 ? 64 : 32);  // query rows per step
  static constexpr bool DQ_T = DQK != 64;           // dQ accumulated transposed (head dims on TMEM lanes)
  static constexpr int DQ_GROUPS = DQK >= 192 ? 2 : 1;
  static constexpr int DQ_GROUP_DIMS = DQK == 192 ? 64 : 128;  // first head dim of group g = g * DQ_GROUP_DIMS
  static constexpr int DQ_N = BQ < 64 ? 64 : BQ;    // columns per dQ^T group (one full 64-wide MN-major atom)
  static constexpr int K_BYTES = BKV * DQK * 2;
  static constexpr int V_BYTES = HAS_DK ? BKV * DV * 2 : 0;
  static constexpr int Q_BYTES = BQ * DQK * 2;      // per stage
  static constexpr int DO_BYTES = BQ * DV * 2;
  static constexpr int PT_BYTES = HAS_DV ? BKV * DQ_N * 2 : 0;   // rows of P^T / dS^T are at least one 128-byte span
  static constexpr int DST_BYTES = HAS_DK ? BKV * DQ_N * 2 : 0;
  static constexpr int SOFT_WARPS = BQ >= 64 ? 8 : 4;
  static constexpr int GROUPS = SOFT_WARPS / 4;        // column halves per key-row quarter
  static constexpr int THREADS = 32 * (SOFT_WARPS + 2);
  // boxes of 32 rows x 128 B, shared out over the warps: eight, or four where shared memory is short
  static constexpr int DQ_STAGE_BYTES = (DQK == 256 && PASS == 2) ? 4 * 4096 : 4 * 2 * 4096;
  static constexpr int SLAB_BYTES = DQ_STAGE_BYTES / SOFT_WARPS;
  static constexpr int STAT_BYTES = SOFT_WARPS * 2 * BQ * 4;  // per softmax warp: lse[BQ] | delta[BQ]
  static constexpr int OFF_K = 0;
  static constexpr int OFF_V = OFF_K + K_BYTES;
  static constexpr int OFF_Q = OFF_V + V_BYTES;           // 2 stages of (Q | dO)
  static constexpr int OFF_PT = OFF_Q + 2 * (Q_BYTES + DO_BYTES);
  static constexpr int OFF_DST = OFF_PT + PT_BYTES;
  static constexpr int OFF_DQ = OFF_DST + DST_BYTES;
  static constexpr int OFF_STAT = OFF_DQ + DQ_STAGE_BYTES;
  static constexpr int OFF_BAR = OFF_STAT + STAT_BYTES;
  static constexpr int SMEM_BYTES = OFF_BAR + 256;
  static constexpr int TMEM_COLS = 512;
  static constexpr int COL_ST = 0, COL_DPT = BQ, COL_DV = 2 * BQ, COL_DK = COL_DV + (HAS_DV ? DV : 0),
                       COL_DQ = COL_DK + (HAS_DK ? DQK : 0);
  static_assert(COL_DQ + (!HAS_DK ? 0 : (DQ_T ? DQ_GROUPS * DQ_N : DQK)) <= TMEM_COLS, "tensor memory budget");
  static_assert(DQK != 256 || PASS != 0, "head_dim 256 runs as two passes");
  static_assert(SMEM_BYTES <= 232448, "shared memory budget");
};

struct BwdArgs {
  int S, H, Hkv, causal, window;
  float scale, softcap;
  const float* lse;
  const float* delta;
  int* status;
};

template <int DQK, int DV, bool CAP, int PASS = 0>
__global__ void __launch_bounds__((BwdCfg<DQK, DV, PASS>::THREADS), 1)
flash_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                 const __grid_constant__ CUtensorMap tmDQ, const __grid_constant__ CUtensorMap tmDK,
                 const __grid_constant__ CUtensorMap tmDV, BwdArgs args) {
  using C = BwdCfg<DQK, DV, PASS>;
  constexpr int BQ = C::BQ;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* k_s = smem + C::OFF_K;
  uint8_t* v_s = smem + C::OFF_V;
  uint8_t* qdo_s = smem + C::OFF_Q;
  uint8_t* pt_s = smem + C::OFF_PT;
  uint8_t* dst_s = smem + C::OFF_DST;
  uint8_t* dq_s = smem + C::OFF_DQ;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::OFF_BAR);
  uint64_t* kv_full = bars + 0;
  uint64_t* qdo_full = bars + 1;   // [2]
  uint64_t* qdo_empty = bars + 3;  // [2]
  uint64_t* st_full = bars + 5;
  uint64_t* pds_full = bars + 6;
  uint64_t* mma2_done = bars + 7;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int j = blockIdx.x;  // key block (small j = most work, scheduled first)
  const int hk = blockIdx.y;
  const int b = blockIdx.z;
  const int G = args.H / args.Hkv;
  const int nQ = args.S / BQ;
  const int key0 = j * BKV;
  const int tok0 = b * args.S;
  const int i_begin = args.causal ? key0 / BQ : 0;
  int i_end = nQ;
  if (args.window > 0) {
    const int last_q = key0 + BKV - 1 + args.window - 1;  // largest query index that still sees this block
    i_end = min(nQ, last_q / BQ + 1);
  }
  const int n_i = max(i_end - i_begin, 0);
  const int n_steps = n_i * G;

  if ((smem_u32(smem) & 1023u) != 0) {
    if (threadIdx.x == 0 && args.status) atomicCAS(args.status, 0, MT_ERR_BAD_ARGS);
    return;
  }
  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&qdo_full[s], 1);
      mbar_init(&qdo_empty[s], 1);
    }
    mbar_init(st_full, 1);
    mbar_init(pds_full, C::SOFT_WARPS);
    mbar_init(mma2_done, 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  constexpr int kTmaWarp = C::SOFT_WARPS, kMmaWarp = C::SOFT_WARPS + 1;
  if (warp == kMmaWarp) {
    tmem_alloc(tmem_slot, C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == kTmaWarp) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      mbar_expect_tx(kv_full, C::K_BYTES + C::V_BYTES);
#pragma unroll
      for (int x = 0; x < DQK / 64; ++x)  // one 64-wide swizzle atom per load
        tma_load_3d(k_s + x * (BKV * 128), &tmK, kv_full, x * 64, hk, tok0 + key0);
      if constexpr (C::HAS_DK) {
#pragma unroll
        for (int x = 0; x < DV / 64; ++x) tma_load_3d(v_s + x * (BKV * 128), &tmV, kv_full, x * 64, hk, tok0 + key0);
      }
      for (int t = 0; t < n_steps; ++t) {
        const int s = t & 1;
        const uint32_t ph = (t >> 1) & 1;
        if (!mbar_wait(&qdo_empty[s], ph ^ 1, abort_flag, args.status, MT_ERR_TIMEOUT_EMPTY)) break;
        const int h = hk * G + t / n_i;
        const int q0 = (i_begin + t % n_i) * BQ;
        uint8_t* q_dst = qdo_s + s * (C::Q_BYTES + C::DO_BYTES);
        mbar_expect_tx(&qdo_full[s], C::Q_BYTES + C::DO_BYTES);
#pragma unroll
        for (int x = 0; x < DQK / 64; ++x)
          tma_load_3d(q_dst + x * (BQ * 128), &tmQ, &qdo_full[s], x * 64, h, tok0 + q0);
#pragma unroll
        for (int x = 0; x < DV / 64; ++x)
          tma_load_3d(q_dst + C::Q_BYTES + x * (BQ * 128), &tmDO, &qdo_full[s], x * 64, h, tok0 + q0);
      }
    }
  } else if (warp == kMmaWarp) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(BKV, BQ, false, false);     // S^T, dP^T
      constexpr uint32_t idesc_dv = make_idesc_bf16(BKV, DV, false, true);     // dV : B = dO as [K=q, N=dv]
      constexpr uint32_t idesc_dk = make_idesc_bf16(BKV, DQK, false, true);    // dK : B = Q as [K=q, N=dqk]
      constexpr uint32_t idesc_dq = C::DQ_T ? make_idesc_bf16(128, C::DQ_N, true, true)  // dQ^T : A = K_j read MN-major
                                            : make_idesc_bf16(BQ, DQK, true, true);      // dQ : A = dS^T read MN-major
      const uint32_t k_addr = smem_u32(k_s), v_addr = smem_u32(v_s);
      const uint32_t pt_addr = smem_u32(pt_s), dst_addr = smem_u32(dst_s);
      bool ok = mbar_wait(kv_full, 0, abort_flag, args.status, MT_ERR_TIMEOUT_FULL);
      auto issue_scores = [&](int t) {
        const uint32_t q_addr = smem_u32(qdo_s + (t & 1) * (C::Q_BYTES + C::DO_BYTES));
        const uint32_t do_addr = q_addr + C::Q_BYTES;
#pragma unroll
        for (int k = 0; k < DQK / 16; ++k)
          tc_mma_f16(tmem_base + C::COL_ST,
                     make_smem_desc_sw128(k_addr + (k >> 2) * (BKV * 128) + (k & 3) * 32, 16, 1024),
                     make_smem_desc_sw128(q_addr + (k >> 2) * (BQ * 128) + (k & 3) * 32, 16, 1024), idesc_s,
                     k != 0 ? 1u : 0u);
        if constexpr (C::HAS_DK) {
#pragma unroll
          for (int k = 0; k < DV / 16; ++k)
            tc_mma_f16(tmem_base + C::COL_DPT,
                       make_smem_desc_sw128(v_addr + (k >> 2) * (BKV * 128) + (k & 3) * 32, 16, 1024),
                       make_smem_desc_sw128(do_addr + (k >> 2) * (BQ * 128) + (k & 3) * 32, 16, 1024), idesc_s,
                       k != 0 ? 1u : 0u);
        }
        tc_commit(st_full);
      };
      if (ok && n_steps > 0) {
        ok = mbar_wait(&qdo_full[0], 0, abort_flag, args.status, MT_ERR_TIMEOUT_FULL);
        if (ok) {
          tc_fence_after_sync();
          issue_scores(0);
        }
      }
      for (int t = 0; t < n_steps && ok; ++t) {
        const int s = t & 1;
        if (!mbar_wait(pds_full, t & 1, abort_flag, args.status, MT_ERR_TIMEOUT_TMEM_EMPTY)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t q_addr = smem_u32(qdo_s + s * (C::Q_BYTES + C::DO_BYTES));
        const uint32_t do_addr = q_addr + C::Q_BYTES;
        // dV += P^T dO ; dK += dS^T Q   (A: [128 keys x 128 queries] K-major in two 64-query atoms)
        if constexpr (C::HAS_DV) {
#pragma unroll
          for (int k = 0; k < BQ / 16; ++k) {
            const uint32_t aoff = (k >> 2) * (BKV * 128) + (k & 3) * 32;
            tc_mma_f16(tmem_base + C::COL_DV, make_smem_desc_sw128(pt_addr + aoff, 16, 1024),
                       make_smem_desc_sw128(do_addr + k * (16 * 128), BQ * 128, 1024), idesc_dv, (t | k) != 0 ? 1u : 0u);
          }
        }
        if constexpr (C::HAS_DK) {
#pragma unroll
          for (int k = 0; k < BQ / 16; ++k) {
            const uint32_t aoff = (k >> 2) * (BKV * 128) + (k & 3) * 32;
            tc_mma_f16(tmem_base + C::COL_DK, make_smem_desc_sw128(dst_addr + aoff, 16, 1024),
                       make_smem_desc_sw128(q_addr + k * (16 * 128), BQ * 128, 1024), idesc_dk, (t | k) != 0 ? 1u : 0u);
          }
        }
        // dQ = dS K : A = dS^T tile read MN-major (M = queries contiguous in 64-wide atoms, K = key rows),
        //             B = K_j tile read MN-major (N = dh contiguous, K = key rows)
#pragma unroll
        for (int k = 0; k < (C::HAS_DK ? BKV / 16 : 0); ++k) {
          const uint64_t d_ds = make_smem_desc_sw128(dst_addr + k * (16 * 128), BKV * 128, 1024);
          if (C::DQ_T) {
#pragma unroll
            for (int g = 0; g < C::DQ_GROUPS; ++g)  // group g covers head dims g * DQ_GROUP_DIMS .. + 127
              tc_mma_f16(tmem_base + C::COL_DQ + g * C::DQ_N,
                         make_smem_desc_sw128(k_addr + g * (C::DQ_GROUP_DIMS / 64) * (BKV * 128) + k * (16 * 128),
                                              BKV * 128, 1024),
                         d_ds, idesc_dq, k != 0 ? 1u : 0u);
          } else {
            tc_mma_f16(tmem_base + C::COL_DQ, d_ds, make_smem_desc_sw128(k_addr + k * (16 * 128), BKV * 128, 1024),
                       idesc_dq, k != 0 ? 1u : 0u);
          }
        }
        tc_commit(&qdo_empty[s]);
        tc_commit(mma2_done);
        if (t + 1 < n_steps) {
          const int s2 = (t + 1) & 1;
          if (!mbar_wait(&qdo_full[s2], ((t + 1) >> 1) & 1, abort_flag, args.status, MT_ERR_TIMEOUT_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          issue_scores(t + 1);
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax backward (thread = key row)
    const int wq = warp & 3;    // lane quarter of tensor memory = 32-key block of this warp
    const int grp = warp >> 2;  // which part of the step's query columns (and of the drain / epilogue boxes)
    const int r = wq * 32 + lane;
    const int kidx = key0 + r;
    const uint32_t t_row = tmem_base + (static_cast<uint32_t>(wq * 32) << 16);
    const float sc = args.scale;
    const float cap = args.softcap;
    uint8_t* dq_stage = dq_s + warp * C::SLAB_BYTES;
    bool ok = true;

    auto drain_dq = [&](int t_prev) {
      const int h = hk * G + t_prev / n_i;
      const int q0 = (i_begin + t_prev % n_i) * BQ;
      if (lane == 0) tma_wait_group_read<0>();
      __syncwarp();
      if constexpr (!C::DQ_T) {
        // dQ partial: TMEM lanes = query rows; this warp owns rows warp*32 .. +31, boxes of 32 dims
#pragma unroll
        for (int c = 0; c < DQK / 32; ++c) {
          if (C::GROUPS == 2 && c != grp) continue;  // one box per warp
          uint32_t v[32];
          tmem_ld_32x32b_x32(t_row + C::COL_DQ + c * 32, v);
          tc_wait_ld();
          uint8_t* srow = dq_stage + (C::GROUPS == 2 ? 0 : c * 4096) + lane * 128;
#pragma unroll
          for (int g = 0; g < 8; ++g) {
            uint4 w = make_uint4(__float_as_uint(__uint_as_float(v[4 * g]) * sc),
                                 __float_as_uint(__uint_as_float(v[4 * g + 1]) * sc),
                                 __float_as_uint(__uint_as_float(v[4 * g + 2]) * sc),
                                 __float_as_uint(__uint_as_float(v[4 * g + 3]) * sc));
            *reinterpret_cast<uint4*>(srow + ((g ^ (lane & 7)) << 4)) = w;
          }
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
#pragma unroll
          for (int c = 0; c < DQK / 32; ++c) {
            if (C::GROUPS == 2 && c != grp) continue;
            tma_reduce_add_3d(&tmDQ, dq_stage + (C::GROUPS == 2 ? 0 : c * 4096), c * 32, h, tok0 + q0 + wq * 32);
          }
          tma_commit_group();
        }
      } else {
        // dQ^T partial: TMEM lanes = head dims (group g: dims 64g + warp*32 + lane), columns = queries.
        // Each box of the reduce-add is [32 queries x 32 dims]: lane d writes element d of every query row.
        constexpr int kSlabBoxes = C::SLAB_BYTES / 4096;
        int box = 0;
#pragma unroll
        for (int g = 0; g < C::DQ_GROUPS; ++g) {
          // overlapping groups (192 dims): lanes 0..63 of the later group repeat dims of the previous one
          if (g > 0 && C::DQ_GROUP_DIMS < 128 && wq < 2) continue;
#pragma unroll
          for (int c = 0; c < BQ / 32; ++c) {
            if (C::GROUPS == 2 && c != grp) continue;  // one box per warp
            if (box >= kSlabBoxes) {  // slab full: the earlier boxes must have been read out
              if (lane == 0) tma_wait_group_read<0>();
              __syncwarp();
            }
            uint32_t v[32];
            tmem_ld_32x32b_x32(t_row + C::COL_DQ + g * C::DQ_N + c * 32, v);
            tc_wait_ld();
            uint8_t* slab = dq_stage + (box % kSlabBoxes) * 4096;
            uint8_t* bx = slab + (lane & 3) * 4;
#pragma unroll
            for (int q = 0; q < 32; ++q)
              *reinterpret_cast<float*>(bx + q * 128 + (((lane >> 2) ^ (q & 7)) << 4)) = __uint_as_float(v[q]) * sc;
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              tma_reduce_add_3d(&tmDQ, slab, C::DQ_GROUP_DIMS * g + wq * 32, h, tok0 + q0 + c * 32);
              tma_commit_group();
            }
            ++box;
          }
        }
      }
    };

    // per-query statistics: each warp keeps a private copy of the step's 128 (lse * log2e, delta) pairs in shared
    // memory (written by its own lanes, read back as 16-byte broadcasts), prefetched one step ahead in registers
    float* stat = reinterpret_cast<float*>(smem + C::OFF_STAT) + warp * (2 * BQ);
    auto load_stats = [&](int t, float4& l4, float4& d4) {
      const int h = hk * G + t / n_i;
      const int q0 = (i_begin + t % n_i) * BQ;
      if (lane * 4 < BQ) {
        const int64_t sbase = (static_cast<int64_t>(b) * args.H + h) * args.S + q0 + lane * 4;
        l4 = *reinterpret_cast<const float4*>(args.lse + sbase);
        d4 = *reinterpret_cast<const float4*>(args.delta + sbase);
      }
    };
    float4 lse_n = make_float4(0.f, 0.f, 0.f, 0.f), delta_n = lse_n;
    if (n_steps > 0) load_stats(0, lse_n, delta_n);
    const float c1 = sc * kLog2e;
    const float sc_over_cap = CAP ? sc / cap : 0.f;
    const float cap_l2 = CAP ? cap * kLog2e : 0.f;

    auto score_block = [&](auto mask_tag, int q0) {
      constexpr bool MASK = decltype(mask_tag)::value;
#pragma unroll
      for (int cc = 0; cc < (BQ / 32) / C::GROUPS; ++cc) {
        const int c = grp * ((BQ / 32) / C::GROUPS) + cc;  // this warp's share of the query columns
        uint32_t sv[32];
        uint32_t dv[32];
        tmem_ld_32x32b_x32(t_row + C::COL_ST + c * 32, sv);
        if constexpr (C::HAS_DK) tmem_ld_32x32b_x32(t_row + C::COL_DPT + c * 32, dv);
        tc_wait_ld();
        float p[32], ds[32];
#pragma unroll
        for (int e4 = 0; e4 < 8; ++e4) {
          const float4 l4 = *reinterpret_cast<const float4*>(stat + c * 32 + e4 * 4);
          const float4 d4 = *reinterpret_cast<const float4*>(stat + BQ + c * 32 + e4 * 4);
          const float lq[4] = {l4.x, l4.y, l4.z, l4.w};
          const float dq4[4] = {d4.x, d4.y, d4.z, d4.w};
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int e = e4 * 4 + u;
            const float x = __uint_as_float(sv[e]);
            float pe, slope = 1.f;
            if constexpr (CAP) {
              const float th = tanhf(x * sc_over_cap);
              pe = exp2f(fmaf(th, cap_l2, -lq[u]));
              slope = 1.f - th * th;
            } else {
              pe = exp2f(fmaf(x, c1, -lq[u]));
            }
            if constexpr (MASK) {
              const int qidx = q0 + c * 32 + e;
              const bool dead = (args.causal && kidx > qidx) || (args.window > 0 && qidx - kidx >= args.window);
              if (dead) pe = 0.f;
            }
            p[e] = pe;
            if constexpr (C::HAS_DK) {
              float d = pe * (__uint_as_float(dv[e]) - dq4[u]);
              if constexpr (CAP) d *= slope;
              ds[e] = d;  // the softmax scale is applied once to dK (epilogue) and dQ (drain)
            }
          }
        }
        uint8_t* prow = pt_s + (c >> 1) * (BKV * 128) + r * 128;
        uint8_t* drow = dst_s + (c >> 1) * (BKV * 128) + r * 128;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          const int chunk = (c & 1) * 4 + g;
          if constexpr (C::HAS_DV) {
            uint4 w;
            w.x = pack_bf16x2(p[8 * g + 0], p[8 * g + 1]);
            w.y = pack_bf16x2(p[8 * g + 2], p[8 * g + 3]);
            w.z = pack_bf16x2(p[8 * g + 4], p[8 * g + 5]);
            w.w = pack_bf16x2(p[8 * g + 6], p[8 * g + 7]);
            *reinterpret_cast<uint4*>(prow + ((chunk ^ (r & 7)) << 4)) = w;
          }
          if constexpr (C::HAS_DK) {
            uint4 d;
            d.x = pack_bf16x2(ds[8 * g + 0], ds[8 * g + 1]);
            d.y = pack_bf16x2(ds[8 * g + 2], ds[8 * g + 3]);
            d.z = pack_bf16x2(ds[8 * g + 4], ds[8 * g + 5]);
            d.w = pack_bf16x2(ds[8 * g + 6], ds[8 * g + 7]);
            *reinterpret_cast<uint4*>(drow + ((chunk ^ (r & 7)) << 4)) = d;
          }
        }
      }
    };

    for (int t = 0; t < n_steps && ok; ++t) {
      const int i = i_begin + t % n_i;
      const int q0 = i * BQ;
      // publish this step's statistics to the warp's slab, then prefetch the next step's
      __syncwarp();
      if (lane * 4 < BQ) {
        reinterpret_cast<float4*>(stat)[lane] =
            make_float4(lse_n.x * kLog2e, lse_n.y * kLog2e, lse_n.z * kLog2e, lse_n.w * kLog2e);
        reinterpret_cast<float4*>(stat + BQ)[lane] = delta_n;
      }
      __syncwarp();
      if (t + 1 < n_steps) load_stats(t + 1, lse_n, delta_n);
      if (!mbar_wait_warp(st_full, t & 1, abort_flag, args.status, MT_ERR_TIMEOUT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after_sync();
      if (t > 0) {
        // previous step's dV/dK/dQ MMAs finished: P^T / dS^T buffers are free and dQ(t-1) can be drained
        if (!mbar_wait_warp(mma2_done, (t - 1) & 1, abort_flag, args.status, MT_ERR_TIMEOUT_TMEM_FULL)) { ok = false; break; }
        tc_fence_after_sync();
        if constexpr (C::HAS_DK) drain_dq(t - 1);
      }
      const bool need_mask = (args.causal && (key0 + BKV - 1 > q0)) ||
                             (args.window > 0 && (q0 + BQ - 1 - key0 >= args.window));
      if (need_mask) score_block(std::true_type{}, q0);
      else score_block(std::false_type{}, q0);
      fence_proxy_async_smem();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(pds_full);
    }
    // tail: last dQ partial, then dK / dV
    if (ok && n_steps > 0) {
      ok = mbar_wait_warp(mma2_done, (n_steps - 1) & 1, abort_flag, args.status, MT_ERR_TIMEOUT_TMEM_FULL);
      if (ok) {
        tc_fence_after_sync();
        if constexpr (C::HAS_DK) drain_dq(n_steps - 1);
      }
    }
    if (ok) {
      if (lane == 0) tma_wait_group_read<0>();
      __syncwarp();
      // dV then dK: this warp's 32 key rows x DH dims (bf16) through its staging slab, one 64-dim box (32 rows of
      // 128 bytes) at a time; the slab holds two boxes
      // with eight warps the first group writes dV and the second dK, each through its one-box slab
      constexpr int kSlabBoxes = C::SLAB_BYTES / 4096;
      int boxes = 0;
#pragma unroll
      for (int which = 0; which < 2; ++which) {
        if (C::GROUPS == 2 && which != grp) continue;
        if ((which == 0 && !C::HAS_DV) || (which == 1 && !C::HAS_DK)) continue;
        const int col = which == 0 ? C::COL_DV : C::COL_DK;
        const float osc = which == 0 ? 1.f : sc;
#pragma unroll
        for (int half = 0; half < (which == 0 ? DV : DQK) / 64; ++half, ++boxes) {
          if (boxes >= kSlabBoxes) {  // slab full: wait until the earlier boxes have been read out
            if (lane == 0) tma_wait_group_read<0>();
            __syncwarp();
          }
          uint8_t* slab = dq_stage + (boxes % kSlabBoxes) * 4096;
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            uint32_t v[32];
            if (n_steps > 0) {
              tmem_ld_32x32b_x32(t_row + col + half * 64 + c * 32, v);
              tc_wait_ld();
            } else {
#pragma unroll
              for (int e = 0; e < 32; ++e) v[e] = 0;
            }
            uint8_t* srow = slab + lane * 128;
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              uint4 w;
              w.x = pack_bf16x2(__uint_as_float(v[8 * g + 0]) * osc, __uint_as_float(v[8 * g + 1]) * osc);
              w.y = pack_bf16x2(__uint_as_float(v[8 * g + 2]) * osc, __uint_as_float(v[8 * g + 3]) * osc);
              w.z = pack_bf16x2(__uint_as_float(v[8 * g + 4]) * osc, __uint_as_float(v[8 * g + 5]) * osc);
              w.w = pack_bf16x2(__uint_as_float(v[8 * g + 6]) * osc, __uint_as_float(v[8 * g + 7]) * osc);
              const int chunk = c * 4 + g;
              *reinterpret_cast<uint4*>(srow + ((chunk ^ (lane & 7)) << 4)) = w;
            }
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_store_3d(which == 0 ? &tmDV : &tmDK, slab, half * 64, hk, tok0 + key0 + wq * 32);
            tma_commit_group();
          }
        }
      }
    }
    if (lane == 0) tma_wait_group<0>();
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == kMmaWarp) {
    tc_fence_after_sync();
    __syncwarp();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

union Pack8 {
  uint4 u;
  __nv_bfloat16 h[8];
};

// delta[b,h,s] = sum_d dO * O over the DV value dims; also clears the fp32 dQ accumulator row (DQK floats).
// DV/8 lanes per (token, head) row.
template <int DQK, int DV>
__global__ void bwd_prepare_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ dout,
                                   float* __restrict__ delta, float* __restrict__ dq_accum, int B, int S, int H,
                                   int64_t o_stride, int64_t do_stride) {
  constexpr int LPR = DV / 8;          // lanes per row, 8 elements each
  constexpr int RPW = 32 / LPR;        // rows per warp pass
  constexpr int ZPL = DQK / LPR;       // dQ floats cleared per lane (8 or 12)
  const int64_t rows = static_cast<int64_t>(B) * S * H;
  const int lane = threadIdx.x & 31;
  const int sub = lane / LPR;
  const int l8 = lane % LPR;
  for (int64_t row = (static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5)) * RPW + sub; row < rows;
       row += static_cast<int64_t>(gridDim.x) * (blockDim.x >> 5) * RPW) {
    const int64_t tok = row / H;
    const int h = static_cast<int>(row % H);
    Pack8 a, g;
    a.u = *reinterpret_cast<const uint4*>(o + tok * o_stride + h * DV + l8 * 8);
    g.u = *reinterpret_cast<const uint4*>(dout + tok * do_stride + h * DV + l8 * 8);
    float s = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) s += __bfloat162float(a.h[e]) * __bfloat162float(g.h[e]);
#pragma unroll
    for (int m = 1; m < LPR; m <<= 1) s += __shfl_xor_sync(0xffffffffu, s, m);
    if (l8 == 0) {
      const int bb = static_cast<int>(tok / S);
      const int ss = static_cast<int>(tok % S);
      delta[(static_cast<int64_t>(bb) * H + h) * S + ss] = s;
    }
    float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
    float4* dq = reinterpret_cast<float4*>(dq_accum + row * DQK + l8 * ZPL);
#pragma unroll
    for (int e = 0; e < ZPL / 4; ++e) dq[e] = z;
  }
}

template <int DH>
__global__ void bwd_finish_kernel(const float* __restrict__ dq_accum, __nv_bfloat16* __restrict__ dq, int64_t tokens,
                                  int H, int64_t dq_stride) {
  const int64_t total = tokens * H * (DH / 8);
  for (int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
       idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int c = static_cast<int>(idx % (DH / 8));
    const int64_t th = idx / (DH / 8);
    const int h = static_cast<int>(th % H);
    const int64_t tok = th / H;
    const float4 a = *reinterpret_cast<const float4*>(dq_accum + th * DH + c * 8);
    const float4 b2 = *reinterpret_cast<const float4*>(dq_accum + th * DH + c * 8 + 4);
    Pack8 o;
    o.h[0] = __float2bfloat16(a.x); o.h[1] = __float2bfloat16(a.y);
    o.h[2] = __float2bfloat16(a.z); o.h[3] = __float2bfloat16(a.w);
    o.h[4] = __float2bfloat16(b2.x); o.h[5] = __float2bfloat16(b2.y);
    o.h[6] = __float2bfloat16(b2.z); o.h[7] = __float2bfloat16(b2.w);
    *reinterpret_cast<uint4*>(dq + tok * dq_stride + h * DH + c * 8) = o.u;
  }
}

template <int DQK, int DV, int PASS>
void launch_pass(const CUtensorMap& tQ, const CUtensorMap& tK, const CUtensorMap& tV, const CUtensorMap& tDO,
                 const CUtensorMap& tDQ, const CUtensorMap& tDK, const CUtensorMap& tDV, const BwdArgs& a, dim3 grid,
                 bool cap, cudaStream_t stream) {
  using C = BwdCfg<DQK, DV, PASS>;
  static bool configured = false;
  if (!configured) {
    MT_CUDA_CHECK(cudaFuncSetAttribute(flash_bwd_kernel<DQK, DV, false, PASS>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES));
    MT_CUDA_CHECK(cudaFuncSetAttribute(flash_bwd_kernel<DQK, DV, true, PASS>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES));
    configured = true;
  }
  if (cap)
    flash_bwd_kernel<DQK, DV, true, PASS><<<grid, C::THREADS, C::SMEM_BYTES, stream>>>(tQ, tK, tV, tDO, tDQ, tDK, tDV, a);
  else
    flash_bwd_kernel<DQK, DV, false, PASS><<<grid, C::THREADS, C::SMEM_BYTES, stream>>>(tQ, tK, tV, tDO, tDQ, tDK, tDV, a);
}

template <int DQK, int DV>
void launch_bwd(const AttnParams& p, int num_sms, cudaStream_t stream) {
  using C = BwdCfg<DQK, DV, DQK == 256 ? 1 : 0>;  // tile sizes are the same in every pass
  constexpr int BQ = C::BQ;
  const auto bf = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const auto sw = CU_TENSOR_MAP_SWIZZLE_128B;
  const uint64_t tokens = static_cast<uint64_t>(p.B) * p.S;
  bwd_prepare_kernel<DQK, DV><<<num_sms * 8, 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(p.o), static_cast<const __nv_bfloat16*>(p.dout), p.delta,
      static_cast<float*>(p.dq_accum), p.B, p.S, p.H, p.o_row_stride, p.do_row_stride);
  CUtensorMap tQ = make_tmap_3d(p.q, bf, 2, tokens, p.H, DQK, p.q_row_stride, DQK, BQ, 1, 64, sw);
  CUtensorMap tK = make_tmap_3d(p.k, bf, 2, tokens, p.Hkv, DQK, p.k_row_stride, DQK, BKV, 1, 64, sw);
  CUtensorMap tV = make_tmap_3d(p.v, bf, 2, tokens, p.Hkv, DV, p.v_row_stride, DV, BKV, 1, 64, sw);
  CUtensorMap tDO = make_tmap_3d(p.dout, bf, 2, tokens, p.H, DV, p.do_row_stride, DV, BQ, 1, 64, sw);
  CUtensorMap tDQ = make_tmap_3d(p.dq_accum, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, tokens, p.H, DQK,
                                 static_cast<uint64_t>(p.H) * DQK, DQK, 32, 1, 32, sw);
  CUtensorMap tDK = make_tmap_3d(p.dk, bf, 2, tokens, p.Hkv, DQK, p.dk_row_stride, DQK, 32, 1, 64, sw);
  CUtensorMap tDV = make_tmap_3d(p.dv, bf, 2, tokens, p.Hkv, DV, p.dv_row_stride, DV, 32, 1, 64, sw);
  BwdArgs a{p.S, p.H, p.Hkv, p.causal, p.window, p.scale, p.softcap, p.lse, p.delta, p.status};
  dim3 grid(p.S / BKV, p.Hkv, p.B);
  static const bool pipelined = [] {  // MT_ATTN_BWD_PIPELINED=0 falls back to the 128-query-step kernel for head_dim 64
    const char* e = std::getenv("MT_ATTN_BWD_PIPELINED");
    return e == nullptr || e[0] != '0';
  }();
  if (DQK == 64 && DV == 64 && pipelined) {
    flash_bwd_pipe64_main(p, stream);  // software-pipelined 64-query steps (flash_bwd_pipe64.cu)
  } else if constexpr (DQK == 256) {
    launch_pass<DQK, DV, 1>(tQ, tK, tV, tDO, tDQ, tDK, tDV, a, grid, p.softcap > 0.f, stream);
    launch_pass<DQK, DV, 2>(tQ, tK, tV, tDO, tDQ, tDK, tDV, a, grid, p.softcap > 0.f, stream);
  } else {
    launch_pass<DQK, DV, 0>(tQ, tK, tV, tDO, tDQ, tDK, tDV, a, grid, p.softcap > 0.f, stream);
  }
  MT_CUDA_CHECK(cudaGetLastError());
  bwd_finish_kernel<DQK><<<num_sms * 8, 256, 0, stream>>>(static_cast<const float*>(p.dq_accum),
                                                          static_cast<__nv_bfloat16*>(p.dq_out),
                                                          static_cast<int64_t>(tokens), p.H, p.dq_row_stride);
  MT_CUDA_CHECK(cudaGetLastError());
}

}  // namespace

// p.dq_accum: fp32 [B*S, H, dh] scratch; p.delta: fp32 [B,H,S] scratch; p.dq_out (bf16) row pitch = dq_row_stride.
void flash_attn_bwd(const AttnParams& p, int num_sms, cudaStream_t stream) {
  if (p.S % 128 != 0) throw std::runtime_error("flash_attn_bwd: sequence length must be a multiple of 128");
  const int dv = p.dv_dim > 0 ? p.dv_dim : p.dh;
  if (p.dh == 64 && dv == 64) launch_bwd<64, 64>(p, num_sms, stream);
  else if (p.dh == 128 && dv == 128) launch_bwd<128, 128>(p, num_sms, stream);
  else if (p.dh == 192 && dv == 128) launch_bwd<192, 128>(p, num_sms, stream);
  else if (p.dh == 256 && dv == 256) launch_bwd<256, 256>(p, num_sms, stream);
  else throw std::runtime_error("flash_attn_bwd: head dims must be 64, 128, 256 or 192/128");
}

}  // namespace mt
