// Causal / sliding-window flash attention forward for sm_100a (bf16, head_dim 64, 128 or 256, grouped-query K/V; also
// the multi-head-latent shape with 192-wide queries/keys and 128-wide values).
//
// One CTA = one (batch, head, 128-query-row block), walking the visible keys in blocks of 64.  Roles:
//   warps 0-3  softmax      : thread r owns query row r.  Reads S = Q K^T from tensor memory (tcgen05.ld) once per
//                             block, forms the probabilities against a lazily updated reference (any value within
//                             2^12 of the row maximum keeps bf16 / fp32 in range; O is rescaled in TMEM only when a row
//                             outgrows it) and writes P (bf16) back INTO TENSOR MEMORY, over the columns its scores
//                             came from; the second MMA takes P from there as its A operand, so P never touches
//                             shared memory.
//   warp 4     TMA producer : Q once, then K and V blocks through two separate 2-stage rings (non-multicast tile
//                             loads).  A K stage is free again as soon as its score MMA has run, long before the V
//                             stage of the same block, which is what lets the scores run one block ahead.
//   warp 5     MMA issuer   : S_b = Q K_i^T (M=128, N=64, K=dh) into one of TWO score buffers and O += P_i V_i
//                             (M=128, N=dv, K=64, A from tensor memory) with tcgen05.mma.  The scores of block i+1
//                             are issued before the softmax of block i has finished, so the tensor pipe works under the
//                             softmax instead of alternating with it: the softmax threads only ever wait for a
//                             score buffer at start-up.
// Tensor memory per CTA: 2 x 64 score / probability columns + dv output columns (256 columns up to dv = 128, so two
// CTAs share an SM and overlap each other's remaining gaps; 512 for head_dim 256).  Shared memory holds Q, two K
// and two V stages.  Blocks above the causal diagonal / outside the window are never loaded.  Output: O (bf16) by
// TMA store (staged in the Q tile's shared memory) and the row-wise log-sum-exp (natural log, of the scaled and
// capped scores) for the backward pass.  Every mbarrier wait is bounded; on expiry an error code is recorded and
// the CTA unwinds.
#include "../common/ptx.cuh"
#include "../common/tmap.h"
#include <type_traits>
#include "../api.h"

namespace mt {
namespace {

constexpr int BLOCK_M = 128;
constexpr int BN = 64;  // keys per block
constexpr int kThreads = 192;
constexpr float kLog2e = 1.4426950408889634f;

template <int DQK, int DV>
struct FwdCfg {
  static constexpr int Q_BYTES = BLOCK_M * DQK * 2;
  static constexpr int K_BYTES = BN * DQK * 2;
  static constexpr int V_BYTES = BN * DV * 2;
  static constexpr int O_STAGE_BYTES = BLOCK_M * DV * 2;  // staged in the Q tile once the last score MMA has run
  static constexpr int SMEM_DATA = Q_BYTES + 2 * K_BYTES + 2 * V_BYTES;
  static constexpr int SMEM_BYTES = SMEM_DATA + 256;
  static constexpr int TMEM_COLS = 2 * BN + DV <= 256 ? 256 : 512;
  static constexpr int S_COL = 0;        // buffer b at S_COL + b * BN; P_b (bf16 pairs) occupies its first BN / 2 columns
  static constexpr int O_COL = 2 * BN;
  static_assert(O_STAGE_BYTES <= Q_BYTES, "the output tile is staged in the query tile's shared memory");
  static_assert(2 * BN + DV <= TMEM_COLS, "accumulators must fit the allocation");
  static_assert(SMEM_BYTES <= 232448, "shared memory budget");
};

struct FwdArgs {
  int S, H, Hkv, causal, window;
  float scale, softcap;
  float* lse;
  int* status;
};

template <int DQK, int DV, bool CAP>
__global__ void __launch_bounds__(kThreads, (FwdCfg<DQK, DV>::TMEM_COLS == 256 && FwdCfg<DQK, DV>::SMEM_BYTES <= 113 * 1024) ? 2 : 1)
flash_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO, FwdArgs args) {
  using C = FwdCfg<DQK, DV>;
  constexpr int QK_ATOMS = DQK / 64;  // 64-element (128 B) swizzle atoms along the head dims
  constexpr int V_ATOMS = DV / 64;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* q_s = smem;
  uint8_t* k_s = q_s + C::Q_BYTES;        // stage s at k_s + s * K_BYTES
  uint8_t* v_s = k_s + 2 * C::K_BYTES;    // stage s at v_s + s * V_BYTES
  uint64_t* bars = reinterpret_cast<uint64_t*>(v_s + 2 * C::V_BYTES);
  uint64_t* q_full = bars + 0;
  uint64_t* k_full = bars + 1;    // [2]
  uint64_t* k_empty = bars + 3;   // [2]
  uint64_t* v_full = bars + 5;    // [2]
  uint64_t* v_empty = bars + 7;   // [2]
  uint64_t* s_full = bars + 9;    // [2]  scores of a block are in buffer b
  uint64_t* p_full = bars + 11;   // [2]  probabilities of a block are in buffer b (four warp arrivals)
  uint64_t* pv_done = bars + 13;  //      O holds every block up to the committed one (one phase per block)
  uint64_t* o_staged = bars + 14;
  uint64_t* o_final = bars + 15;  //      the last block's second MMA has completed (single phase)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
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
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 1);
      mbar_init(&s_full[s], 1);
      mbar_init(&p_full[s], 4);
    }
    mbar_init(pv_done, 1);
    mbar_init(o_staged, 4);
    mbar_init(o_final, 1);
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
      auto load_k = [&](int i) -> bool {
        const int s = i & 1;
        if (!mbar_wait(&k_empty[s], ((i >> 1) & 1) ^ 1, abort_flag, args.status, MT_ERR_TIMEOUT_EMPTY)) return false;
        mbar_expect_tx(&k_full[s], C::K_BYTES);
        const int key0 = tok0 + (j_begin + i) * BN;
#pragma unroll
        for (int a = 0; a < QK_ATOMS; ++a)
          tma_load_3d(k_s + s * C::K_BYTES + a * (BN * 128), &tmK, &k_full[s], a * 64, hk, key0);
        return true;
      };
      auto load_v = [&](int i) -> bool {
        const int s = i & 1;
        if (!mbar_wait(&v_empty[s], ((i >> 1) & 1) ^ 1, abort_flag, args.status, MT_ERR_TIMEOUT_EMPTY)) return false;
        mbar_expect_tx(&v_full[s], C::V_BYTES);
        const int key0 = tok0 + (j_begin + i) * BN;
#pragma unroll
        for (int a = 0; a < V_ATOMS; ++a)
          tma_load_3d(v_s + s * C::V_BYTES + a * (BN * 128), &tmV, &v_full[s], a * 64, hk, key0);
        return true;
      };
      // K runs one block ahead of V: K(i+1) is requested before V(i), so a wait for a V stage (freed by the second
      // MMA of two blocks earlier) never holds back the K block that the next score MMA needs
      bool ok = n_blocks > 0 ? load_k(0) : true;
      for (int i = 0; i < n_blocks && ok; ++i) {
        if (i + 1 < n_blocks) ok = load_k(i + 1);
        if (ok) ok = load_v(i);
      }
    }
  } else if (warp == 5) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_qk = make_idesc_bf16(BLOCK_M, BN, false, false);
      constexpr uint32_t idesc_pv = make_idesc_bf16(BLOCK_M, DV, false, true);  // A: P from tensor memory (K-major)
      const uint32_t q_addr = smem_u32(q_s);
      bool ok = mbar_wait(q_full, 0, abort_flag, args.status, MT_ERR_TIMEOUT_FULL);
      auto issue_qk = [&](int i) -> bool {  // scores of block i into buffer i & 1
        const int s = i & 1;
        if (!mbar_wait(&k_full[s], (i >> 1) & 1, abort_flag, args.status, MT_ERR_TIMEOUT_FULL)) return false;
        tc_fence_after_sync();
        const uint32_t k_addr = smem_u32(k_s + s * C::K_BYTES);
#pragma unroll
        for (int k = 0; k < DQK / 16; ++k) {
          const uint32_t off = (k >> 2) * (BLOCK_M * 128) + (k & 3) * 32;
          const uint32_t koff = (k >> 2) * (BN * 128) + (k & 3) * 32;
          tc_mma_f16(tmem_base + C::S_COL + s * BN, make_smem_desc_sw128(q_addr + off, 16, 1024),
                     make_smem_desc_sw128(k_addr + koff, 16, 1024), idesc_qk, k != 0 ? 1u : 0u);
        }
        tc_commit(&k_empty[s]);
        tc_commit(&s_full[s]);
        return true;
      };
      if (ok && n_blocks > 0) ok = issue_qk(0);
      if (ok && n_blocks > 1) ok = issue_qk(1);
      for (int i = 0; i < n_blocks && ok; ++i) {
        const int s = i & 1;
        const uint32_t ph = (i >> 1) & 1;
        // P(i) is in tensor memory (and O has been rescaled if it had to be); V(i) has landed
        if (!mbar_wait(&p_full[s], ph, abort_flag, args.status, MT_ERR_TIMEOUT_TMEM_EMPTY)) { ok = false; break; }
        if (!mbar_wait(&v_full[s], ph, abort_flag, args.status, MT_ERR_TIMEOUT_FULL)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t v_addr = smem_u32(v_s + s * C::V_BYTES);
        const uint32_t p_tmem = tmem_base + C::S_COL + s * BN;
#pragma unroll
        for (int k = 0; k < BN / 16; ++k)  // 16 keys = 8 columns of packed bf16 pairs in tensor memory
          tc_mma_f16_ts(tmem_base + C::O_COL, p_tmem + k * 8,
                        make_smem_desc_sw128(v_addr + k * (16 * 128), BN * 128, 1024), idesc_pv, (i | k) != 0 ? 1u : 0u);
        tc_commit(&v_empty[s]);
        tc_commit(pv_done);
        if (i == n_blocks - 1) tc_commit(o_final);
        // the tensor pipe executes in issue order: the scores of block i+2 overwrite buffer s only after P(i) was read
        if (i + 2 < n_blocks) ok = issue_qk(i + 2);
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax + epilogue (thread = query row)
    const int r = threadIdx.x;  // 0..127
    const int q_idx = q0 + r;
    const uint32_t t_row = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
    // running maximum is tracked on the raw scores (scaling and tanh capping are monotone), the reference M_l2 and the
    // running sum live in log2 units of the transformed score
    float m_raw = -INFINITY, M_l2 = 0.f, l_run = 0.f;
    const float c1 = args.scale * kLog2e;
    const float sc_over_cap = CAP ? args.scale / args.softcap : 0.f;
    const float cap_l2 = CAP ? args.softcap * kLog2e : 0.f;
    // The reference only has to keep the exponentials in range (bf16 and fp32 share the exponent width), not to
    // equal the running maximum: it moves (and O is rescaled) only when some row of the warp outgrows it by more
    // than kSlack (log2 units) or had no live key so far.
    constexpr float kSlack = 12.f;
    bool ok = true;

    auto softmax_block = [&](auto mask_tag, int i) -> bool {
      constexpr bool MASK = decltype(mask_tag)::value;
      const int key0 = (j_begin + i) * BN;
      const uint32_t s_col = t_row + C::S_COL + (i & 1) * BN;
      float x[BN];
#pragma unroll
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32b_x32(s_col + c * 32, v);
        tc_wait_ld();
#pragma unroll
        for (int e = 0; e < 32; ++e) x[c * 32 + e] = __uint_as_float(v[e]);
      }
      float m_blk = -INFINITY;
#pragma unroll
      for (int e = 0; e < BN; ++e) {
        if constexpr (MASK) {
          const int kidx = key0 + e;
          const bool dead = (args.causal && kidx > q_idx) || (args.window > 0 && q_idx - kidx >= args.window);
          if (dead) x[e] = -INFINITY;
        }
        m_blk = fmaxf(m_blk, x[e]);
      }
      bool grow = false;
      if (m_blk != -INFINITY) {
        const float t_blk = CAP ? cap_l2 * tanhf(m_blk * sc_over_cap) : m_blk * c1;
        grow = (m_raw == -INFINITY) || (t_blk - M_l2 > kSlack);
      }
      if (__any_sync(0xffffffffu, grow)) {
        float alpha = 1.f;
        if (grow) {
          const float m_new = fmaxf(m_raw, m_blk);
          const float M_new = CAP ? cap_l2 * tanhf(m_new * sc_over_cap) : m_new * c1;
          alpha = (m_raw == -INFINITY) ? 0.f : exp2f(M_l2 - M_new);
          M_l2 = M_new;
          l_run *= alpha;
        }
        if (i > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
          // O must hold every earlier block before it is rescaled; the second MMA of THIS block cannot start before
          // this warp has arrived on p_full, so the accumulator is quiet in between.  The parity wait is sound here:
          // the scores of block i were issued behind the second MMA of block i-2, so at this point pv_done has
          // completed i-1 or i phases, never fewer (a waiter two phases behind would read a stale parity).
          if (!mbar_wait_warp(pv_done, (i - 1) & 1, abort_flag, args.status, MT_ERR_TIMEOUT_TMEM_FULL)) return false;
          tc_fence_after_sync();
#pragma unroll
          for (int c = 0; c < DV / 32; ++c) {
            uint32_t o[32];
            tmem_ld_32x32b_x32(t_row + C::O_COL + c * 32, o);
            tc_wait_ld();
#pragma unroll
            for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * alpha);
            tmem_st_32x32b_x32(t_row + C::O_COL + c * 32, o);
          }
        }
      }
      m_raw = fmaxf(m_raw, m_blk);
      // probabilities (masked scores are -inf and give exactly 0), packed to bf16 pairs, back into the score columns
      float l_blk = 0.f;
#pragma unroll
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t w[16];
#pragma unroll
        for (int e = 0; e < 32; e += 2) {
          float p0, p1;
          if constexpr (CAP) {
            p0 = exp2f(fmaf(tanhf(x[c * 32 + e] * sc_over_cap), cap_l2, -M_l2));
            p1 = exp2f(fmaf(tanhf(x[c * 32 + e + 1] * sc_over_cap), cap_l2, -M_l2));
            if constexpr (MASK) {  // tanh(-inf) = -1 is finite: masked entries need an explicit zero
              if (x[c * 32 + e] == -INFINITY) p0 = 0.f;
              if (x[c * 32 + e + 1] == -INFINITY) p1 = 0.f;
            }
          } else {
            p0 = exp2f(fmaf(x[c * 32 + e], c1, -M_l2));
            p1 = exp2f(fmaf(x[c * 32 + e + 1], c1, -M_l2));
          }
          l_blk += p0 + p1;
          w[e >> 1] = pack_bf16x2(p0, p1);
        }
        tmem_st_32x32b_x16(s_col + c * 16, w);
      }
      l_run += l_blk;
      tc_wait_st();
      return true;
    };

    for (int i = 0; i < n_blocks && ok; ++i) {
      const int key0 = (j_begin + i) * BN;
      if (!mbar_wait_warp(&s_full[i & 1], (i >> 1) & 1, abort_flag, args.status, MT_ERR_TIMEOUT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after_sync();
      const bool need_mask = (args.causal && (key0 + BN - 1 > q0)) ||
                             (args.window > 0 && (key0 <= q0 + BLOCK_M - 1 - args.window));
      ok = need_mask ? softmax_block(std::true_type{}, i) : softmax_block(std::false_type{}, i);
      if (!ok) break;
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[i & 1]);
    }
    // epilogue: O / l -> bf16 -> staging (the Q tile: every score MMA has completed by now) -> TMA store ; lse
    // (its own single-phase barrier: after the last softmax block pv_done may still be two phases short, where a
    // parity wait would pass on the stale phase)
    if (ok && n_blocks > 0) ok = mbar_wait_warp(o_final, 0, abort_flag, args.status, MT_ERR_TIMEOUT_TMEM_FULL);
    if (ok) {
      tc_fence_after_sync();
      const float inv_l = l_run > 0.f ? 1.f / l_run : 0.f;
      uint8_t* stage = q_s;  // staging rows are 128 B (64 bf16) per atom
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
          (l_run > 0.f) ? (M_l2 / kLog2e + logf(l_run)) : -INFINITY;
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
  CUtensorMap tK = make_tmap_3d(p.k, bf, 2, tokens, p.Hkv, DQK, p.k_row_stride, DQK, BN, 1, 64, sw);
  CUtensorMap tV = make_tmap_3d(p.v, bf, 2, tokens, p.Hkv, DV, p.v_row_stride, DV, BN, 1, 64, sw);
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
