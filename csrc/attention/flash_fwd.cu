// Causal / sliding-window flash attention forward for sm_100a (bf16, head_dim 64, 128 or 256, grouped-query K/V; also
// the multi-head-latent shape with 192-wide queries/keys and 128-wide values).
//
// One CTA = one (batch, head, 128-query-row block).  Roles:
//   warps 0-3  softmax      : thread r owns query row r.  Reads S = Q K^T from tensor memory (tcgen05.ld) ONCE per
//                             block: probabilities are formed against a lazily updated reference (any value within
//                             2^12 of the row maximum keeps bf16 / fp32 in range), the row maximum is tracked on the
//                             side, and only when a row outgrows the reference is O rescaled in TMEM and the block
//                             redone.  P (bf16) goes to 128B-swizzled shared memory as the A operand of the second MMA.
//   warp 4     TMA producer : Q once, then K/V blocks through a 2-stage ring (non-multicast tile loads).
//   warp 5     MMA issuer   : S = Q K^T (M=128, N=BN, K=dh) and O += P V (M=128, N=dh, K=BN) with tcgen05.mma,
//                             accumulators in TMEM (S: BN columns, O: dh columns -> 256 columns per CTA).
// Two CTAs fit on an SM (112 KB shared memory, 256 TMEM columns each), so one CTA's softmax overlaps the other
// CTA's MMAs.  Blocks above the causal diagonal / outside the window are never loaded.  Output: O (bf16) by TMA
// store and the row-wise log-sum-exp (natural log, of the scaled and capped scores) for the backward pass.
// Every mbarrier wait is bounded; on expiry an error code is recorded and the CTA unwinds.
#include "../common/ptx.cuh"
#include "../common/tmap.h"
#include <type_traits>
#include "../api.h"

namespace mt {
namespace {

constexpr int BLOCK_M = 128;
constexpr int kThreads = 192;
constexpr float kLog2e = 1.4426950408889634f;

template <int DQK, int DV>
struct FwdCfg {
  static constexpr int BN = (DQK == 64) ? 128 : 64;
  static constexpr int Q_BYTES = BLOCK_M * DQK * 2;
  static constexpr int K_BYTES = BN * DQK * 2;
  static constexpr int V_BYTES = BN * DV * 2;
  static constexpr int P_BYTES = BLOCK_M * BN * 2;
  static constexpr int O_STAGE_BYTES = BLOCK_M * DV * 2;  // reuses the P region, or the K/V ring when larger
  static constexpr int SMEM_DATA = Q_BYTES + 2 * (K_BYTES + V_BYTES) + P_BYTES;
  static constexpr int SMEM_BYTES = SMEM_DATA + 256;
  static constexpr int TMEM_COLS = BN + DV <= 256 ? 256 : 512;  // head_dim 256: one CTA per SM, all of tensor memory
  static constexpr int S_COL = 0;
  static constexpr int O_COL = BN;
  static_assert(BN + DV <= TMEM_COLS, "accumulators must fit the allocation");
  static_assert(O_STAGE_BYTES <= P_BYTES || O_STAGE_BYTES <= 2 * (K_BYTES + V_BYTES), "output staging");
};

struct FwdArgs {
  int S, H, Hkv, causal, window;
  float scale, softcap;
  float* lse;
  int* status;
};

template <int DQK, int DV, bool CAP>
__global__ void __launch_bounds__(kThreads, 2)
flash_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO, FwdArgs args) {
  using C = FwdCfg<DQK, DV>;
  constexpr int BN = C::BN;
  constexpr int QK_ATOMS = DQK / 64;  // 64-element (128 B) swizzle atoms along the head dims
  constexpr int V_ATOMS = DV / 64;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* q_s = smem;
  uint8_t* kv_s = q_s + C::Q_BYTES;  // stage s: K at kv_s + s*(K+V), V right after K
  uint8_t* p_s = kv_s + 2 * (C::K_BYTES + C::V_BYTES);
  uint64_t* bars = reinterpret_cast<uint64_t*>(p_s + C::P_BYTES);
  uint64_t* q_full = bars + 0;
  uint64_t* kv_full = bars + 1;    // [2]
  uint64_t* kv_empty = bars + 3;   // [2]
  uint64_t* s_full = bars + 5;
  uint64_t* p_full = bars + 6;
  uint64_t* pv_done = bars + 7;
  uint64_t* o_staged = bars + 8;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 9);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_qb = args.S / BLOCK_M;
  const int qb = num_qb - 1 - blockIdx.x;  // heavy (late) blocks first
  const int h = blockIdx.y;
  const int b = blockIdx.z;
  const int hk = h / (args.H / args.Hkv);
  const int q0 = qb * BLOCK_M;
  const int tok0 = b * args.S;

  // key-block range of this query block
  int j_end = args.causal ? (q0 + BLOCK_M + BN - 1) / BN : args.S / BN;
  if (j_end > args.S / BN) j_end = args.S / BN;
  int j_begin = 0;
  if (args.window > 0) {
    const int first_key = q0 - args.window + 1;
    if (first_key > 0) j_begin = first_key / BN;
  }
  const int n_blocks = j_end - j_begin;

  if ((smem_u32(smem) & 1023u) != 0) {  // swizzled tiles need 1024-byte alignment
    if (threadIdx.x == 0 && args.status) atomicCAS(args.status, 0, MT_ERR_BAD_ARGS);
    return;
  }
  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(p_full, 4);
    mbar_init(pv_done, 1);
    mbar_init(o_staged, 4);
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tmap(&tmQ);
    prefetch_tmap(&tmK);
    prefetch_tmap(&tmV);
    prefetch_tmap(&tmO);
  }
  if (warp == 5) {
    tmem_alloc(tmem_slot, C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 4) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      mbar_expect_tx(q_full, C::Q_BYTES);
#pragma unroll
      for (int a = 0; a < QK_ATOMS; ++a)
        tma_load_3d(q_s + a * (BLOCK_M * 128), &tmQ, q_full, a * 64, h, tok0 + q0);
      for (int i = 0; i < n_blocks; ++i) {
        const int s = i & 1;
        const uint32_t ph = (i >> 1) & 1;
        if (!mbar_wait(&kv_empty[s], ph ^ 1, abort_flag, args.status, MT_ERR_TIMEOUT_EMPTY)) break;
        uint8_t* k_dst = kv_s + s * (C::K_BYTES + C::V_BYTES);
        uint8_t* v_dst = k_dst + C::K_BYTES;
        mbar_expect_tx(&kv_full[s], C::K_BYTES + C::V_BYTES);
        const int key0 = tok0 + (j_begin + i) * BN;
#pragma unroll
        for (int a = 0; a < QK_ATOMS; ++a) tma_load_3d(k_dst + a * (BN * 128), &tmK, &kv_full[s], a * 64, hk, key0);
#pragma unroll
        for (int a = 0; a < V_ATOMS; ++a) tma_load_3d(v_dst + a * (BN * 128), &tmV, &kv_full[s], a * 64, hk, key0);
      }
    }
  } else if (warp == 5) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_qk = make_idesc_bf16(BLOCK_M, BN, false, false);
      constexpr uint32_t idesc_pv = make_idesc_bf16(BLOCK_M, DV, false, true);
      const uint32_t q_addr = smem_u32(q_s);
      const uint32_t p_addr = smem_u32(p_s);
      bool ok = mbar_wait(q_full, 0, abort_flag, args.status, MT_ERR_TIMEOUT_FULL);
      auto issue_qk = [&](int i) {
        const uint32_t k_addr = smem_u32(kv_s + (i & 1) * (C::K_BYTES + C::V_BYTES));
#pragma unroll
        for (int k = 0; k < DQK / 16; ++k) {
          const uint32_t off = (k >> 2) * (BLOCK_M * 128) + (k & 3) * 32;
          const uint32_t koff = (k >> 2) * (BN * 128) + (k & 3) * 32;
          tc_mma_f16(tmem_base + C::S_COL, make_smem_desc_sw128(q_addr + off, 16, 1024),
                     make_smem_desc_sw128(k_addr + koff, 16, 1024), idesc_qk, k != 0 ? 1u : 0u);
        }
        tc_commit(s_full);
      };
      if (ok && n_blocks > 0) {
        ok = mbar_wait(&kv_full[0], 0, abort_flag, args.status, MT_ERR_TIMEOUT_FULL);
        if (ok) {
          tc_fence_after_sync();
          issue_qk(0);
        }
      }
      for (int i = 0; i < n_blocks && ok; ++i) {
        const int s = i & 1;
        // P(i) is in shared memory and O has been rescaled
        if (!mbar_wait(p_full, i & 1, abort_flag, args.status, MT_ERR_TIMEOUT_TMEM_EMPTY)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t v_addr = smem_u32(kv_s + s * (C::K_BYTES + C::V_BYTES) + C::K_BYTES);
#pragma unroll
        for (int k = 0; k < BN / 16; ++k) {
          const uint32_t poff = (k >> 2) * (BLOCK_M * 128) + (k & 3) * 32;
          tc_mma_f16(tmem_base + C::O_COL, make_smem_desc_sw128(p_addr + poff, 16, 1024),
                     make_smem_desc_sw128(v_addr + k * (16 * 128), BN * 128, 1024), idesc_pv,
                     (i | k) != 0 ? 1u : 0u);
        }
        tc_commit(&kv_empty[s]);
        tc_commit(pv_done);
        if (i + 1 < n_blocks) {
          const int s2 = (i + 1) & 1;
          if (!mbar_wait(&kv_full[s2], ((i + 1) >> 1) & 1, abort_flag, args.status, MT_ERR_TIMEOUT_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          issue_qk(i + 1);
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax + epilogue (thread = query row)
    const int r = threadIdx.x;  // 0..127
    const int q_idx = q0 + r;
    const uint32_t t_row = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
    // running maximum is tracked on the raw scores (scaling and tanh capping are monotone), the running sum on
    // exp2 of (transformed score - transformed max) in log2 units
    float m_raw = -INFINITY, M_l2 = -INFINITY, l_run = 0.f;
    const float c1 = args.scale * kLog2e;
    const float sc_over_cap = CAP ? args.scale / args.softcap : 0.f;
    const float cap_l2 = CAP ? args.softcap * kLog2e : 0.f;
    bool ok = true;

    // One pass over a score block: probabilities relative to the reference `M_ref` (log2 units) -> bf16 -> swizzled
    // shared memory; returns their sum and, with TRACK, the block's raw row maximum.
    auto exp_pass = [&](auto mask_tag, auto track_tag, int i, float M_ref, float& m_blk) -> float {
      constexpr bool MASK = decltype(mask_tag)::value;
      constexpr bool TRACK = decltype(track_tag)::value;
      const int key0 = (j_begin + i) * BN;
      float l_blk = 0.f;
      constexpr int kUnroll = BN == 128 ? 2 : 1;  // measured: more unrolling spills, less exposes the load latency
#pragma unroll kUnroll
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32b_x32(t_row + C::S_COL + c * 32, v);
        tc_wait_ld();
        float p[32];
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          const float x = __uint_as_float(v[e]);
          float pe;
          if constexpr (CAP) pe = exp2f(fmaf(tanhf(x * sc_over_cap), cap_l2, -M_ref));
          else pe = exp2f(fmaf(x, c1, -M_ref));
          if constexpr (MASK) {
            const int kidx = key0 + c * 32 + e;
            const bool dead = (args.causal && kidx > q_idx) || (args.window > 0 && q_idx - kidx >= args.window);
            if (dead) pe = 0.f;
            if constexpr (TRACK) m_blk = fmaxf(m_blk, dead ? -INFINITY : x);
          } else {
            if constexpr (TRACK) m_blk = fmaxf(m_blk, x);
          }
          p[e] = pe;
          l_blk += pe;
        }
        uint8_t* prow = p_s + (c >> 1) * (BLOCK_M * 128) + r * 128;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          uint4 w;
          w.x = pack_bf16x2(p[8 * g + 0], p[8 * g + 1]);
          w.y = pack_bf16x2(p[8 * g + 2], p[8 * g + 3]);
          w.z = pack_bf16x2(p[8 * g + 4], p[8 * g + 5]);
          w.w = pack_bf16x2(p[8 * g + 6], p[8 * g + 7]);
          const int chunk = (c & 1) * 4 + g;
          *reinterpret_cast<uint4*>(prow + ((chunk ^ (r & 7)) << 4)) = w;
        }
      }
      return l_blk;
    };

    // The softmax reference M_l2 only has to keep the exponentials in range (bf16 and fp32 share the exponent width),
    // not to equal the running maximum.  After the first block a block is therefore processed in ONE pass against the
    // current reference while its maximum is tracked on the side; only when some row of the warp outgrows the
    // reference by more than kSlack (log2 units), or had no live key so far, the reference moves, O is rescaled
    // and the block's probabilities are recomputed.
    constexpr float kSlack = 12.f;
    auto softmax_block = [&](auto mask_tag, int i) -> bool {
      constexpr bool MASK = decltype(mask_tag)::value;
      const int key0 = (j_begin + i) * BN;
      float m_blk = -INFINITY;
      if (i > 0) {
        // O(i-1) has landed (its MMAs precede this block's score MMA): P may be overwritten and O rescaled
        if (!mbar_wait_warp(pv_done, (i - 1) & 1, abort_flag, args.status, MT_ERR_TIMEOUT_TMEM_FULL)) return false;
        tc_fence_after_sync();
        const float l_blk = exp_pass(mask_tag, std::true_type{}, i, M_l2, m_blk);
        bool grow = false;
        if (m_blk != -INFINITY) {
          const float t_blk = CAP ? cap_l2 * tanhf(m_blk * sc_over_cap) : m_blk * c1;
          grow = (m_raw == -INFINITY) || (t_blk - M_l2 > kSlack);
        }
        if (!__any_sync(0xffffffffu, grow)) {
          l_run += l_blk;
          return true;
        }
      } else {
        // first block: row maximum of the raw scores
#pragma unroll
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t v[32];
          tmem_ld_32x32b_x32(t_row + C::S_COL + c * 32, v);
          tc_wait_ld();
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            float x = __uint_as_float(v[e]);
            if constexpr (MASK) {
              const int kidx = key0 + c * 32 + e;
              const bool dead = (args.causal && kidx > q_idx) || (args.window > 0 && q_idx - kidx >= args.window);
              if (dead) x = -INFINITY;
            }
            m_blk = fmaxf(m_blk, x);
          }
        }
      }
      const float m_new = fmaxf(m_raw, m_blk);
      float M_new;
      if (m_new == -INFINITY) M_new = 0.f;
      else M_new = CAP ? cap_l2 * tanhf(m_new * sc_over_cap) : m_new * c1;
      const float alpha = (m_raw == -INFINITY) ? 0.f : exp2f(M_l2 - M_new);
      if (i > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll
        for (int c = 0; c < DV / 32; ++c) {
          uint32_t o[32];
          tmem_ld_32x32b_x32(t_row + C::O_COL + c * 32, o);
          tc_wait_ld();
#pragma unroll
          for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * alpha);
          tmem_st_32x32b_x32(t_row + C::O_COL + c * 32, o);
        }
        tc_wait_st();
      }
      float unused = 0.f;
      const float l_blk = exp_pass(mask_tag, std::false_type{}, i, M_new, unused);
      l_run = l_run * alpha + l_blk;
      m_raw = m_new;
      M_l2 = M_new;
      return true;
    };

    for (int i = 0; i < n_blocks && ok; ++i) {
      const int key0 = (j_begin + i) * BN;
      if (!mbar_wait_warp(s_full, i & 1, abort_flag, args.status, MT_ERR_TIMEOUT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after_sync();
      const bool need_mask = (args.causal && (key0 + BN - 1 > q0)) ||
                             (args.window > 0 && (key0 <= q0 + BLOCK_M - 1 - args.window));
      ok = need_mask ? softmax_block(std::true_type{}, i) : softmax_block(std::false_type{}, i);
      if (!ok) break;
      fence_proxy_async_smem();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
    }
    const float m_run = (m_raw == -INFINITY) ? -INFINITY : M_l2 / kLog2e;
    // epilogue: O / l -> bf16 -> staging (P region) -> TMA store ; lse
    if (ok && n_blocks > 0) {
      ok = mbar_wait_warp(pv_done, (n_blocks - 1) & 1, abort_flag, args.status, MT_ERR_TIMEOUT_TMEM_FULL);
    }
    if (ok) {
      tc_fence_after_sync();
      const float inv_l = l_run > 0.f ? 1.f / l_run : 0.f;
      // staging rows are 128 B (64 bf16) per atom: the P region when it is large enough, else the K/V ring
      uint8_t* stage = (C::P_BYTES >= C::O_STAGE_BYTES) ? p_s : kv_s;
#pragma unroll
      for (int c = 0; c < DV / 32; ++c) {
        uint32_t o[32];
        if (n_blocks > 0) {
          tmem_ld_32x32b_x32(t_row + C::O_COL + c * 32, o);
          tc_wait_ld();
        } else {
#pragma unroll
          for (int e = 0; e < 32; ++e) o[e] = 0;
        }
        uint8_t* orow = stage + (c >> 1) * (BLOCK_M * 128) + r * 128;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          uint4 w;
          w.x = pack_bf16x2(__uint_as_float(o[8 * g + 0]) * inv_l, __uint_as_float(o[8 * g + 1]) * inv_l);
          w.y = pack_bf16x2(__uint_as_float(o[8 * g + 2]) * inv_l, __uint_as_float(o[8 * g + 3]) * inv_l);
          w.z = pack_bf16x2(__uint_as_float(o[8 * g + 4]) * inv_l, __uint_as_float(o[8 * g + 5]) * inv_l);
          w.w = pack_bf16x2(__uint_as_float(o[8 * g + 6]) * inv_l, __uint_as_float(o[8 * g + 7]) * inv_l);
          const int chunk = (c & 1) * 4 + g;
          *reinterpret_cast<uint4*>(orow + ((chunk ^ (r & 7)) << 4)) = w;
        }
      }
      args.lse[(static_cast<int64_t>(b) * args.H + h) * args.S + q_idx] =
          (l_run > 0.f) ? (m_run + logf(l_run)) : -INFINITY;
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(o_staged);
      // all four warps staged their rows -> one thread stores the tile (bounded wait, never a bar.sync that a
      // warp on the error path would skip)
      if (threadIdx.x == 0 && mbar_wait(o_staged, 0, abort_flag, args.status, MT_ERR_TIMEOUT_TMEM_FULL)) {
#pragma unroll
        for (int a = 0; a < V_ATOMS; ++a) tma_store_3d(&tmO, stage + a * (BLOCK_M * 128), a * 64, h, tok0 + q0);
        tma_commit_group();
        tma_wait_group<0>();
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 5) {
    tc_fence_after_sync();
    __syncwarp();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

template <int DQK, int DV, bool CAP>
void launch_fwd(const AttnParams& p, cudaStream_t stream) {
  using C = FwdCfg<DQK, DV>;
  const auto bf = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const auto sw = CU_TENSOR_MAP_SWIZZLE_128B;
  const uint64_t tokens = static_cast<uint64_t>(p.B) * p.S;
  CUtensorMap tQ = make_tmap_3d(p.q, bf, 2, tokens, p.H, DQK, p.q_row_stride, DQK, BLOCK_M, 1, 64, sw);
  CUtensorMap tK = make_tmap_3d(p.k, bf, 2, tokens, p.Hkv, DQK, p.k_row_stride, DQK, C::BN, 1, 64, sw);
  CUtensorMap tV = make_tmap_3d(p.v, bf, 2, tokens, p.Hkv, DV, p.v_row_stride, DV, C::BN, 1, 64, sw);
  CUtensorMap tO = make_tmap_3d(p.o, bf, 2, tokens, p.H, DV, p.o_row_stride, DV, BLOCK_M, 1, 64, sw);
  auto kern = flash_fwd_kernel<DQK, DV, CAP>;
  static bool configured = false;
  if (!configured) {
    MT_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES));
    configured = true;
  }
  FwdArgs a{p.S, p.H, p.Hkv, p.causal, p.window, p.scale, p.softcap, p.lse, p.status};
  dim3 grid(p.S / BLOCK_M, p.H, p.B);
  kern<<<grid, kThreads, C::SMEM_BYTES, stream>>>(tQ, tK, tV, tO, a);
  MT_CUDA_CHECK(cudaGetLastError());
}

}  // namespace

void flash_attn_fwd(const AttnParams& p, int num_sms, cudaStream_t stream) {
  (void)num_sms;
  if (p.S % BLOCK_M != 0) throw std::runtime_error("flash_attn_fwd: sequence length must be a multiple of 128");
  const bool cap = p.softcap > 0.f;
  const int dv = p.dv_dim > 0 ? p.dv_dim : p.dh;
  if (p.dh == 64 && dv == 64) cap ? launch_fwd<64, 64, true>(p, stream) : launch_fwd<64, 64, false>(p, stream);
  else if (p.dh == 128 && dv == 128) cap ? launch_fwd<128, 128, true>(p, stream) : launch_fwd<128, 128, false>(p, stream);
  else if (p.dh == 192 && dv == 128) cap ? launch_fwd<192, 128, true>(p, stream) : launch_fwd<192, 128, false>(p, stream);
  else if (p.dh == 256 && dv == 256) cap ? launch_fwd<256, 256, true>(p, stream) : launch_fwd<256, 256, false>(p, stream);
  else throw std::runtime_error("flash_attn_fwd: head dims must be 64, 128, 256 or 192/128");
}

}  // namespace mt
