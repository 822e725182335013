// Flash attention backward for head_dim 64 with the score and gradient phases software-pipelined inside the CTA.
//
// Same decomposition as flash_bwd.cu (one CTA = one batch, kv head and 128-key block; S^T = K Q^T, dP^T = V dO^T,
// dV += P^T dO, dK += dS^T Q, dQ = dS K), but the queries are walked 64 at a time and the score accumulators, the
// P^T / dS^T tiles in shared memory and the dQ accumulator are all double-buffered:
//     tensor memory (512 columns): S^T[2] 64+64 | dP^T[2] 64+64 | dV 64 | dK 64 | dQ[2] 64+64
// so the MMA warp issues the scores of step t+1 *before* the gradient MMAs of step t, and the eight softmax warps
// work on step t+1 while the tensor cores are still busy with step t; the dQ partial of step t drains while step
// t+1 is in flight.  dQ of a 64-query step is an M = 64 MMA: its accumulator rows sit in lanes 0-15 of each
// 32-lane quarter of tensor memory (row m -> lane 32 (m / 16) + m % 16), which is what the drain reads.
// Roles: warps 0-7 softmax / drain / epilogue (warp & 3 = 32-key lane quarter, warp >> 2 = which 32 of the step's 64
// query columns), warp 8 TMA producer (three Q / dO stages), warp 9 MMA issuer.  All mbarrier waits are bounded.
#include "../common/ptx.cuh"
#include "../common/tmap.h"
#include <type_traits>
#include "../api.h"

namespace mt {
namespace {

constexpr int BKV = 128, BQ = 64, DH = 64;
constexpr int kSoftWarps = 8;
constexpr int kThreads = 32 * (kSoftWarps + 2);
constexpr int kQStages = 3;
constexpr float kLog2e = 1.4426950408889634f;

struct PCfg {
  static constexpr int K_BYTES = BKV * DH * 2;           // 16 KB
  static constexpr int V_BYTES = BKV * DH * 2;
  static constexpr int Q_BYTES = BQ * DH * 2;            // 8 KB
  static constexpr int DO_BYTES = BQ * DH * 2;
  static constexpr int QDO_BYTES = Q_BYTES + DO_BYTES;
  static constexpr int PT_BYTES = BKV * BQ * 2;          // 16 KB: one 128-byte row of 64 queries per key
  static constexpr int SLAB_BYTES = 4096;                // per softmax warp: two 2 KB dQ boxes, or one dV / dK box
  static constexpr int STAT_BYTES = kSoftWarps * 2 * BQ * 4;
  static constexpr int OFF_K = 0;
  static constexpr int OFF_V = OFF_K + K_BYTES;
  static constexpr int OFF_QDO = OFF_V + V_BYTES;
  static constexpr int OFF_PT = OFF_QDO + kQStages * QDO_BYTES;
  static constexpr int OFF_DST = OFF_PT + 2 * PT_BYTES;
  static constexpr int OFF_SLAB = OFF_DST + 2 * PT_BYTES;
  static constexpr int OFF_STAT = OFF_SLAB + kSoftWarps * SLAB_BYTES;
  static constexpr int OFF_BAR = OFF_STAT + STAT_BYTES;
  static constexpr int SMEM_BYTES = OFF_BAR + 256;
  static constexpr int TMEM_COLS = 512;
  static constexpr int COL_ST = 0, COL_DPT = 128, COL_DV = 256, COL_DK = 320, COL_DQ = 384;  // [2] x 64 where doubled
  static_assert(SMEM_BYTES <= 232448, "shared memory budget");
};

struct PArgs {
  int S, H, Hkv, causal, window;
  float scale, softcap;
  const float* lse;
  const float* delta;
  int* status;
};

template <bool CAP>
__global__ void __launch_bounds__(kThreads, 1)
flash_bwd_pipe64_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                        const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                        const __grid_constant__ CUtensorMap tmDQ, const __grid_constant__ CUtensorMap tmDK,
                        const __grid_constant__ CUtensorMap tmDV, PArgs args) {
  using C = PCfg;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* k_s = smem + C::OFF_K;
  uint8_t* v_s = smem + C::OFF_V;
  uint8_t* qdo_s = smem + C::OFF_QDO;
  uint8_t* pt_s = smem + C::OFF_PT;    // [2]
  uint8_t* dst_s = smem + C::OFF_DST;  // [2]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::OFF_BAR);
  uint64_t* kv_full = bars + 0;
  uint64_t* qdo_full = bars + 1;    // [3]
  uint64_t* qdo_empty = bars + 4;   // [3]
  uint64_t* st_full = bars + 7;     // [2]
  uint64_t* pds_full = bars + 9;    // [2], 8 arrivals
  uint64_t* mma2_done = bars + 11;  // [2]
  uint64_t* dq_free = bars + 13;    // [2], 8 arrivals
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int j = blockIdx.x;
  const int hk = blockIdx.y;
  const int b = blockIdx.z;
  const int G = args.H / args.Hkv;
  const int nQ = args.S / BQ;
  const int key0 = j * BKV;
  const int tok0 = b * args.S;
  const int i_begin = args.causal ? key0 / BQ : 0;
  int i_end = nQ;
  if (args.window > 0) {
    const int last_q = key0 + BKV - 1 + args.window - 1;
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
    for (int s = 0; s < kQStages; ++s) {
      mbar_init(&qdo_full[s], 1);
      mbar_init(&qdo_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&st_full[s], 1);
      mbar_init(&pds_full[s], kSoftWarps);
      mbar_init(&mma2_done[s], 1);
      mbar_init(&dq_free[s], kSoftWarps);
    }
    *abort_flag = 0;
    fence_barrier_init();
  }
  constexpr int kTmaWarp = kSoftWarps, kMmaWarp = kSoftWarps + 1;
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
      tma_load_3d(k_s, &tmK, kv_full, 0, hk, tok0 + key0);
      tma_load_3d(v_s, &tmV, kv_full, 0, hk, tok0 + key0);
      for (int t = 0; t < n_steps; ++t) {
        const int s = t % kQStages;
        if (!mbar_wait(&qdo_empty[s], ((t / kQStages) & 1) ^ 1, abort_flag, args.status, MT_ERR_TIMEOUT_EMPTY)) break;
        const int h = hk * G + t / n_i;
        const int q0 = (i_begin + t % n_i) * BQ;
        uint8_t* q_dst = qdo_s + s * C::QDO_BYTES;
        mbar_expect_tx(&qdo_full[s], C::QDO_BYTES);
        tma_load_3d(q_dst, &tmQ, &qdo_full[s], 0, h, tok0 + q0);
        tma_load_3d(q_dst + C::Q_BYTES, &tmDO, &qdo_full[s], 0, h, tok0 + q0);
      }
    }
  } else if (warp == kMmaWarp) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(BKV, BQ, false, false);   // S^T, dP^T : M = keys, N = 64 queries
      constexpr uint32_t idesc_g = make_idesc_bf16(BKV, DH, false, true);    // dV, dK : B = dO / Q as [K = q, N = dh]
      constexpr uint32_t idesc_q = make_idesc_bf16(BQ, DH, true, true);      // dQ : M = 64 queries, A = dS^T MN-major
      const uint32_t k_addr = smem_u32(k_s), v_addr = smem_u32(v_s);
      const uint64_t dk_km = make_smem_desc_sw128(k_addr, 16, 1024), dv_km = make_smem_desc_sw128(v_addr, 16, 1024);
      const uint64_t dk_mn = make_smem_desc_sw128(k_addr, BKV * 128, 1024);
      bool ok = mbar_wait(kv_full, 0, abort_flag, args.status, MT_ERR_TIMEOUT_FULL);
      auto issue_scores = [&](int t) -> bool {
        const int s = t % kQStages;
        if (!mbar_wait(&qdo_full[s], (t / kQStages) & 1, abort_flag, args.status, MT_ERR_TIMEOUT_FULL)) return false;
        tc_fence_after_sync();
        const uint32_t q_addr = smem_u32(qdo_s + s * C::QDO_BYTES);
        const uint32_t do_addr = q_addr + C::Q_BYTES;
        const uint32_t col = (t & 1) * BQ;
        // descriptors differ only in their 16-byte-granular start address (low bits): one add per MMA
        const uint64_t dq = make_smem_desc_sw128(q_addr, 16, 1024), ddo = make_smem_desc_sw128(do_addr, 16, 1024);
#pragma unroll
        for (int k = 0; k < DH / 16; ++k)
          tc_mma_f16(tmem_base + C::COL_ST + col, dk_km + k * 2, dq + k * 2, idesc_s, k != 0 ? 1u : 0u);
#pragma unroll
        for (int k = 0; k < DH / 16; ++k)
          tc_mma_f16(tmem_base + C::COL_DPT + col, dv_km + k * 2, ddo + k * 2, idesc_s, k != 0 ? 1u : 0u);
        tc_commit(&st_full[t & 1]);
        return true;
      };
      if (ok && n_steps > 0) ok = issue_scores(0);
      for (int t = 0; t < n_steps && ok; ++t) {
        // the score buffers of parity (t+1)&1 were last read by the softmax warps in step t-1, whose pds_full this
        // thread waited for in the previous iteration: they are free
        if (t + 1 < n_steps && !issue_scores(t + 1)) { ok = false; break; }
        const int bsel = t & 1;
        if (!mbar_wait(&pds_full[bsel], (t >> 1) & 1, abort_flag, args.status, MT_ERR_TIMEOUT_TMEM_EMPTY)) { ok = false; break; }
        if (t >= 2 && !mbar_wait(&dq_free[bsel], ((t - 2) >> 1) & 1, abort_flag, args.status, MT_ERR_TIMEOUT_TMEM_EMPTY)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const int s = t % kQStages;
        const uint32_t q_addr = smem_u32(qdo_s + s * C::QDO_BYTES);
        const uint32_t do_addr = q_addr + C::Q_BYTES;
        const uint32_t pt_addr = smem_u32(pt_s + bsel * C::PT_BYTES);
        const uint32_t dst_addr = smem_u32(dst_s + bsel * C::PT_BYTES);
        const uint64_t dpt = make_smem_desc_sw128(pt_addr, 16, 1024), dds = make_smem_desc_sw128(dst_addr, 16, 1024);
        const uint64_t ddo_mn = make_smem_desc_sw128(do_addr, BQ * 128, 1024), dq_mn = make_smem_desc_sw128(q_addr, BQ * 128, 1024);
        const uint64_t dds_mn = make_smem_desc_sw128(dst_addr, BKV * 128, 1024);
#pragma unroll
        for (int k = 0; k < BQ / 16; ++k)  // dV += P^T dO : contraction over the 64 queries (16 rows = 2048 B per step)
          tc_mma_f16(tmem_base + C::COL_DV, dpt + k * 2, ddo_mn + k * 128, idesc_g, (t | k) != 0 ? 1u : 0u);
#pragma unroll
        for (int k = 0; k < BQ / 16; ++k)  // dK += dS^T Q
          tc_mma_f16(tmem_base + C::COL_DK, dds + k * 2, dq_mn + k * 128, idesc_g, (t | k) != 0 ? 1u : 0u);
#pragma unroll
        for (int k = 0; k < BKV / 16; ++k)  // dQ = dS K : contraction over the 128 keys, M = 64 queries
          tc_mma_f16(tmem_base + C::COL_DQ + bsel * DH, dds_mn + k * 128, dk_mn + k * 128, idesc_q, k != 0 ? 1u : 0u);
        tc_commit(&qdo_empty[s]);
        tc_commit(&mma2_done[bsel]);
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax backward, dQ drain, epilogue
    const int wq = warp & 3;
    const int grp = warp >> 2;
    const int r = wq * 32 + lane;  // key row of this thread
    const int kidx = key0 + r;
    const uint32_t t_row = tmem_base + (static_cast<uint32_t>(wq * 32) << 16);
    const float sc = args.scale;
    const float cap = args.softcap;
    uint8_t* slab = smem + C::OFF_SLAB + warp * C::SLAB_BYTES;
    float* stat = reinterpret_cast<float*>(smem + C::OFF_STAT) + warp * (2 * BQ);
    bool ok = true;

    auto step_coords = [&](int t, int& h, int& q0) {
      h = hk * G + t / n_i;
      q0 = (i_begin + t % n_i) * BQ;
    };
    auto load_stats = [&](int t, float4& l4, float4& d4) {
      int h, q0;
      step_coords(t, h, q0);
      if (lane * 4 < BQ) {
        const int64_t sbase = (static_cast<int64_t>(b) * args.H + h) * args.S + q0 + lane * 4;
        l4 = *reinterpret_cast<const float4*>(args.lse + sbase);
        d4 = *reinterpret_cast<const float4*>(args.delta + sbase);
      }
    };
    // dQ partial of step tp: an M = 64 accumulator, rows 16 wq .. +15 in lanes 0-15 of this warp's quarter; this warp
    // takes head dims grp*32 .. +31 -> one [16 queries x 32 dims] fp32 box for the TMA reduce-add
    auto drain_dq = [&](int tp) {
      int h, q0;
      step_coords(tp, h, q0);
      uint8_t* box = slab + (tp & 1) * 2048;
      if (lane == 0) tma_wait_group_read<1>();  // the box written two drains ago has been read
      __syncwarp();
      uint32_t v[32];
      tmem_ld_32x32b_x32(t_row + C::COL_DQ + (tp & 1) * DH + grp * 32, v);
      tc_wait_ld();
      if (lane < 16) {
        uint8_t* srow = box + lane * 128;
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          *reinterpret_cast<uint4*>(srow + ((g ^ (lane & 7)) << 4)) = make_uint4(v[4 * g], v[4 * g + 1], v[4 * g + 2], v[4 * g + 3]);
        }
      }
      fence_proxy_async_smem();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        tma_reduce_add_3d(&tmDQ, box, grp * 32, h, tok0 + q0 + wq * 16);
        tma_commit_group();
        mbar_arrive(&dq_free[tp & 1]);  // the accumulator has been read out
      }
    };

    float4 lse_n = make_float4(0.f, 0.f, 0.f, 0.f), delta_n = lse_n;
    if (n_steps > 0) load_stats(0, lse_n, delta_n);
    const float c1 = sc * kLog2e;
    const float sc_over_cap = CAP ? sc / cap : 0.f;
    const float cap_l2 = CAP ? cap * kLog2e : 0.f;

    auto score_block = [&](auto mask_tag, int t, int q0) {
      constexpr bool MASK = decltype(mask_tag)::value;
      const int bsel = t & 1;
      const int c0 = grp * 32;  // this warp's 32 of the step's 64 query columns
      uint32_t sv[32];
      uint32_t dv[32];
      tmem_ld_32x32b_x32(t_row + C::COL_ST + bsel * BQ + c0, sv);
      tmem_ld_32x32b_x32(t_row + C::COL_DPT + bsel * BQ + c0, dv);
      tc_wait_ld();
      float p[32], ds[32];
#pragma unroll
      for (int e4 = 0; e4 < 8; ++e4) {
        const float4 l4 = *reinterpret_cast<const float4*>(stat + c0 + e4 * 4);
        const float4 d4 = *reinterpret_cast<const float4*>(stat + BQ + c0 + e4 * 4);
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
            const int qidx = q0 + c0 + e;
            const bool dead = (args.causal && kidx > qidx) || (args.window > 0 && qidx - kidx >= args.window);
            if (dead) pe = 0.f;
          }
          p[e] = pe;
          // dS carries the softmax scale: (dP - delta) * scale is one FMA against the pre-scaled delta
          float d = pe * fmaf(__uint_as_float(dv[e]), sc, -dq4[u]);
          if constexpr (CAP) d *= slope;
          ds[e] = d;
        }
      }
      uint8_t* prow = pt_s + bsel * C::PT_BYTES + r * 128;
      uint8_t* drow = dst_s + bsel * C::PT_BYTES + r * 128;
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        uint4 w, d;
        w.x = pack_bf16x2(p[8 * g + 0], p[8 * g + 1]);
        w.y = pack_bf16x2(p[8 * g + 2], p[8 * g + 3]);
        w.z = pack_bf16x2(p[8 * g + 4], p[8 * g + 5]);
        w.w = pack_bf16x2(p[8 * g + 6], p[8 * g + 7]);
        d.x = pack_bf16x2(ds[8 * g + 0], ds[8 * g + 1]);
        d.y = pack_bf16x2(ds[8 * g + 2], ds[8 * g + 3]);
        d.z = pack_bf16x2(ds[8 * g + 4], ds[8 * g + 5]);
        d.w = pack_bf16x2(ds[8 * g + 6], ds[8 * g + 7]);
        const int chunk = grp * 4 + g;
        *reinterpret_cast<uint4*>(prow + ((chunk ^ (r & 7)) << 4)) = w;
        *reinterpret_cast<uint4*>(drow + ((chunk ^ (r & 7)) << 4)) = d;
      }
    };

    for (int t = 0; t < n_steps && ok; ++t) {
      int h, q0;
      step_coords(t, h, q0);
      __syncwarp();
      if (lane * 4 < BQ) {
        reinterpret_cast<float4*>(stat)[lane] =
            make_float4(lse_n.x * kLog2e, lse_n.y * kLog2e, lse_n.z * kLog2e, lse_n.w * kLog2e);
        reinterpret_cast<float4*>(stat + BQ)[lane] =
            make_float4(delta_n.x * sc, delta_n.y * sc, delta_n.z * sc, delta_n.w * sc);
      }
      __syncwarp();
      if (t + 1 < n_steps) load_stats(t + 1, lse_n, delta_n);
      if (!mbar_wait_warp(&st_full[t & 1], (t >> 1) & 1, abort_flag, args.status, MT_ERR_TIMEOUT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after_sync();
      // P^T / dS^T of parity t&1 were read by the gradient MMAs of step t-2, whose completion this warp observed
      // when it drained dQ(t-2) in the previous iteration
      const bool need_mask = (args.causal && (key0 + BKV - 1 > q0)) ||
                             (args.window > 0 && (q0 + BQ - 1 - key0 >= args.window));
      if (need_mask) score_block(std::true_type{}, t, q0);
      else score_block(std::false_type{}, t, q0);
      fence_proxy_async_smem();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&pds_full[t & 1]);
      if (t > 0) {  // dQ of the previous step: its MMAs ran while this step's scores were processed
        if (!mbar_wait_warp(&mma2_done[(t - 1) & 1], ((t - 1) >> 1) & 1, abort_flag, args.status, MT_ERR_TIMEOUT_TMEM_FULL)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        drain_dq(t - 1);
      }
    }
    if (ok && n_steps > 0) {
      ok = mbar_wait_warp(&mma2_done[(n_steps - 1) & 1], ((n_steps - 1) >> 1) & 1, abort_flag, args.status,
                          MT_ERR_TIMEOUT_TMEM_FULL);
      if (ok) {
        tc_fence_after_sync();
        drain_dq(n_steps - 1);
      }
    }
    if (ok) {
      if (lane == 0) tma_wait_group_read<0>();
      __syncwarp();
      // dV (first warp group) and dK (second): this warp's 32 key rows x 64 dims as one 4 KB box
      const int col = grp == 0 ? C::COL_DV : C::COL_DK;
      constexpr float osc = 1.f;  // dS already carries the softmax scale
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t v[32];
        if (n_steps > 0) {
          tmem_ld_32x32b_x32(t_row + col + c * 32, v);
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
          *reinterpret_cast<uint4*>(srow + (((c * 4 + g) ^ (lane & 7)) << 4)) = w;
        }
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        tma_store_3d(grp == 0 ? &tmDV : &tmDK, slab, 0, hk, tok0 + key0 + wq * 32);
        tma_commit_group();
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

}  // namespace

// Main kernel only: the caller runs the delta / dQ-clearing pre-pass before and the fp32 -> bf16 dQ pass after.
void flash_bwd_pipe64_main(const AttnParams& p, cudaStream_t stream) {
  using C = PCfg;
  const auto bf = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const auto sw = CU_TENSOR_MAP_SWIZZLE_128B;
  const uint64_t tokens = static_cast<uint64_t>(p.B) * p.S;
  CUtensorMap tQ = make_tmap_3d(p.q, bf, 2, tokens, p.H, DH, p.q_row_stride, DH, BQ, 1, 64, sw);
  CUtensorMap tK = make_tmap_3d(p.k, bf, 2, tokens, p.Hkv, DH, p.k_row_stride, DH, BKV, 1, 64, sw);
  CUtensorMap tV = make_tmap_3d(p.v, bf, 2, tokens, p.Hkv, DH, p.v_row_stride, DH, BKV, 1, 64, sw);
  CUtensorMap tDO = make_tmap_3d(p.dout, bf, 2, tokens, p.H, DH, p.do_row_stride, DH, BQ, 1, 64, sw);
  CUtensorMap tDQ = make_tmap_3d(p.dq_accum, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, tokens, p.H, DH,
                                 static_cast<uint64_t>(p.H) * DH, DH, 16, 1, 32, sw);
  CUtensorMap tDK = make_tmap_3d(p.dk, bf, 2, tokens, p.Hkv, DH, p.dk_row_stride, DH, 32, 1, 64, sw);
  CUtensorMap tDV = make_tmap_3d(p.dv, bf, 2, tokens, p.Hkv, DH, p.dv_row_stride, DH, 32, 1, 64, sw);
  static bool configured = false;
  if (!configured) {
    MT_CUDA_CHECK(cudaFuncSetAttribute(flash_bwd_pipe64_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES));
    MT_CUDA_CHECK(cudaFuncSetAttribute(flash_bwd_pipe64_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES));
    configured = true;
  }
  PArgs a{p.S, p.H, p.Hkv, p.causal, p.window, p.scale, p.softcap, p.lse, p.delta, p.status};
  dim3 grid(p.S / BKV, p.Hkv, p.B);
  if (p.softcap > 0.f) flash_bwd_pipe64_kernel<true><<<grid, kThreads, C::SMEM_BYTES, stream>>>(tQ, tK, tV, tDO, tDQ, tDK, tDV, a);
  else flash_bwd_pipe64_kernel<false><<<grid, kThreads, C::SMEM_BYTES, stream>>>(tQ, tK, tV, tDO, tDQ, tDK, tDV, a);
  MT_CUDA_CHECK(cudaGetLastError());
}

}  // namespace mt
