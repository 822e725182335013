// Host-callable launchers of every CUDA kernel in this tree (plain C++ signatures, no torch types).
// All launchers enqueue on `stream` and return immediately; none allocates device memory.
#pragma once
#include <cuda_runtime.h>
#include <cstdint>

namespace mt {

// ---- gemm/dense_bf16.cu
void gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, int64_t lda, int64_t ldb, int64_t ldc,
               bool a_mn_major, bool b_mn_major, bool out_f32, bool accumulate, int* status, int num_sms,
               cudaStream_t stream);

// ---- gemm/grouped_bf16.cu
// Rows of X / Y are grouped by expert: expert e owns rows offsets[e] .. offsets[e+1], every offset a multiple of 128
// (groups are padded with zero rows).  `offsets` is a device int32[E+1]; M_cap is the allocated row count.
// Y[rows, N] = X[rows, K] * W[e], W = [E, K, N] (w_mn_major) or [E, N, K] (K-major, the data-gradient product).
void grouped_gemm_bf16(const void* X, const void* W, void* Y, const int* offsets, int E, int M_cap, int N, int K,
                       bool w_mn_major, int* status, int num_sms, cudaStream_t stream);
// Per-expert weight gradient: dW[e] (+)= X_e^T @ G_e, X [M_cap, K], G [M_cap, N], dW [E, K, N] fp32 or bf16.
// Experts without rows are skipped (clear dW beforehand when not accumulating).
void grouped_wgrad_bf16(const void* X, const void* G, void* dW, const int* offsets, int E, int M_cap, int N, int K,
                        bool out_f32, bool accumulate, int* status, int num_sms, cudaStream_t stream);
// Kernel choice for this thread's next grouped launches: 0 = default, 1 = single-CTA tiles (128 x 256), 2 = CTA pairs
// (256 x 256).  Shapes the pair kernels do not cover fall back to the single-CTA kernels either way.
void set_grouped_variant(int variant);
// the same two products on CTA pairs (gemm/grouped_bf16_2cta.cu); the functions above route to these by default
void grouped_gemm_bf16_pair(const void* X, const void* W, void* Y, const int* offsets, int E, int M_cap, int N, int K,
                            bool w_mn_major, int* status, int num_sms, cudaStream_t stream);
// Forward product whose output row r goes to the address row_dst[r] (possibly in a peer GPU's memory; 0 = dropped)
void grouped_gemm_scatter_bf16_pair(const void* X, const void* W, const unsigned long long* row_dst, const int* offsets,
                                    int E, int M_cap, int N, int K, bool w_mn_major, int* status, int num_sms,
                                    cudaStream_t stream);
void grouped_wgrad_bf16_pair(const void* X, const void* G, void* dW, const int* offsets, int E, int M_cap, int N, int K,
                             bool out_f32, bool accumulate, int* status, int num_sms, cudaStream_t stream);

// ---- elementwise/rmsnorm.cu
// y = (x [+ residual]) * rsqrt(mean(.^2) + eps) -> bf16, then * w(bf16-rounded).  If residual_out != null the
// pre-norm sum is written there (bf16).  rstd (fp32 per row) is saved for backward.
void rmsnorm_fwd(const void* x, const void* residual, const float* w, void* y, void* residual_out, float* rstd,
                 int64_t rows, int dim, float eps, cudaStream_t stream);
// dx = rstd * (w*dy - xhat * mean(xhat * w*dy)) [+ dres];  dw_partial[blocks, dim] holds per-block sums of dy*xhat.
void rmsnorm_bwd(const void* x, const float* w, const float* rstd, const void* dy, const void* dres, void* dx,
                 float* dw_partial, int num_partials, int64_t rows, int dim, cudaStream_t stream);
void rmsnorm_bwd_reduce(const float* dw_partial, int num_partials, int dim, float* dw, bool accumulate,
                        cudaStream_t stream);

// ---- elementwise/rope.cu
// In-place rotation of the first rot_dim entries of every head of x [tokens, heads, head_dim] (row pitch
// `row_stride` elements) by cos/sin tables [max_pos, rot_dim/2]; positions int32[tokens] or null (= t % seq_len).
void rope_inplace(void* x, const float* cos_t, const float* sin_t, const int* positions, int64_t tokens, int seq_len,
                  int heads, int head_dim, int rot_dim, int64_t row_stride, bool interleave, bool inverse,
                  cudaStream_t stream);

// Half-rotation, out of place (src may equal dst), 16-byte vectors: needs rot_dim % 16 == 0, head_dim % 8 == 0 and
// 16-byte aligned rows.  Columns past rot_dim are copied through.
void rope_apply(const void* src, void* dst, const float* cos_t, const float* sin_t, const int* positions,
                int64_t tokens, int seq_len, int heads, int head_dim, int rot_dim, int64_t src_stride,
                int64_t dst_stride, bool inverse, cudaStream_t stream);

// ---- elementwise/swiglu.cu
// act: 0 silu, 1 gelu(tanh), 2 gelu(erf), 3 relu.  gate/up are column halves [rows, 2*inter] -> out [rows, inter]
void gated_act_fwd(const void* gate_up, void* out, int64_t rows, int inter, int act, cudaStream_t stream);
void gated_act_bwd(const void* gate_up, const void* dout, void* dgate_up, int64_t rows, int inter, int act,
                   cudaStream_t stream);
// out = x * f(gate), f = sigmoid (mode 0) or silu (mode 1); x / gate rows at pitches xs / gs elements
void gate_mul_fwd(const void* x, const void* gate, void* out, int64_t rows, int dim, int64_t xs, int64_t gs, int mode,
                  cudaStream_t stream);
void gate_mul_bwd(const void* x, const void* gate, const void* dout, void* dx, void* dgate, int64_t rows, int dim,
                  int64_t xs, int64_t gs, int mode, cudaStream_t stream);

// ---- elementwise/cross_entropy.cu
// logits bf16 [rows, V] (row pitch ldl) -> per-row loss, z-loss, lse; overwrites logits with dlogits * grad_scale.
void cross_entropy_fwd_bwd(void* logits, const int64_t* targets, float* loss, float* zloss, float* lse,
                           int64_t rows, int V, int64_t ldl, float label_smoothing, float z_weight,
                           float softcap, float grad_scale, bool write_grad, cudaStream_t stream);

// ---- elementwise/threefry.cu
// out[i] = randint element (start + i) of the stream keyed by the two split keys (a0,a1) and (b0,b1), in [0, span)
void threefry_randint(int64_t* out, int64_t count, uint32_t a0, uint32_t a1, uint32_t b0, uint32_t b1, uint64_t start,
                      uint32_t span, cudaStream_t stream);

// ---- elementwise/embedding.cu
void embedding_fwd(const void* table, const int64_t* ids, void* out, int64_t tokens, int dim, float scale, int64_t vocab,
                   cudaStream_t stream);
void embedding_bwd(const void* dout, const int64_t* ids, float* dtable, int64_t tokens, int dim, float scale, int64_t vocab,
                   cudaStream_t stream);

// ---- optim/adamw.cu
// One fused AdamW step over a flat shard: reads grad (bf16 or fp32), updates fp32 master/m/v, writes the bf16
// compute copy.  grad_scale folds 1/accum and the global-norm clip factor (read from device scalar if non-null).
void adamw_step(float* master, float* m, float* v, const void* grad, bool grad_f32, void* param_bf16, int64_t n,
                float lr, float b1, float b2, float eps, float wd, float bc1, float bc2, float grad_scale,
                const float* clip_coef, cudaStream_t stream);
void sumsq(const void* x, bool is_f32, int64_t n, float* out_accum, cudaStream_t stream);

// ---- comm/rs_optim.cu : sharded optimizer step over peer memory (pointers of every rank's symmetric buffer)
constexpr int kMaxPeers = 8;
struct PeerPtrs {
  void* p[kMaxPeers];
};
void symm_barrier(const PeerPtrs& flags, int rank, int world, int seq, int* status, cudaStream_t stream);
// dst[r * n_bytes + i] = shards[r][lo_bytes + r * rank_stride_bytes + i] for every rank r (byte offsets / sizes,
// multiples of 16): an all-gather by plain peer loads (parameter-sharded engine mode: stride 0, every rank's slice
// sits at the same offset of its shard buffer; Muon's publication: stride = slice size, rank r's slice sits at
// its place in the flat buffer)
void peer_gather(const PeerPtrs& shards, int world, int64_t lo_bytes, int64_t rank_stride_bytes, int64_t n_bytes, void* dst,
                 int blocks, cudaStream_t stream);
// out[0..n) = sum over ranks of grads[r][lo..lo+n) ; *sumsq += |out|^2   (n multiple of 4, lo multiple of 4)
void grad_pull_reduce(const PeerPtrs& grads, int rank, int world, int64_t lo, int64_t n, float* out, float* sumsq,
                      cudaStream_t stream);
// One bucket of the same reduction, with the readiness handshake folded in (see comm/rs_optim.cu).  `flags` are the
// ranks' int[world * kBucketSlots] tables; `lo`/`n` select this rank's slice of the bucket in the flat buffers; the
// consumed source elements are cleared on every rank when `clear` is set.  `blocks` caps the grid (<= 0: full device).
constexpr int kBucketSlots = 1024;
void grad_pull_bucket(const PeerPtrs& grads, const PeerPtrs& flags, int rank, int world, int bucket, int seq, int64_t lo,
                      int64_t n, float* out, bool accumulate, bool clear, bool handshake, int blocks, int* status,
                      cudaStream_t stream);
// The handshake alone (one warp): post `seq` for `bucket` to every peer and wait for theirs; a reduction launched
// behind it on the same stream passes handshake = false
void bucket_ready(const PeerPtrs& flags, int rank, int world, int bucket, int seq, int* status, cudaStream_t stream);
// AdamW on the local shard, bf16 result stored to params[r][lo..lo+n) of every rank r   (n multiple of 8)
void adamw_publish(float* master, float* m, float* v, const float* grad, const PeerPtrs& params, int world, int64_t lo,
                   int64_t n, float lr, float b1, float b2, float eps, float wd, float bc1, float bc2,
                   float grad_scale, const float* clip_coef, cudaStream_t stream);

// ---- comm/ep_rows.cu : expert-parallel dispatch (push) / combine (pull) of token rows over peer memory
void ep_push_rows(const void* src, const int* dst_rank, const int64_t* dst_pos, const PeerPtrs& bufs, int64_t rows,
                  int dim, int64_t cap_rows, int* overflow, cudaStream_t stream);
void ep_pull_rows(void* out, const int* src_rank, const int64_t* src_pos, const PeerPtrs& bufs, int64_t rows, int dim,
                  int64_t cap_rows, cudaStream_t stream);
// out[r] = scale[r] (or 1) * row at byte address row_src[r] (peer-mapped or local), zero row where the address is 0
void ep_gather_rows(void* out, const unsigned long long* row_src, const float* row_scale, int64_t rows, int dim,
                    cudaStream_t stream);
// Routing plan of the peer-memory expert exchange (comm/ep_rows.cu).  Count tables are int[2][kMaxPeers][ep_count_slots()]
// in symmetric memory.
int ep_count_slots();
void ep_push_counts(const int64_t* counts, const PeerPtrs& tables, int rank, int R, int E, int parity, cudaStream_t stream);
void ep_plan(const int64_t* flat, const int64_t* pos_l, const int* off_l, const float* w, const int* table, int rank, int R,
             int E, int El, int64_t cap, int K, int64_t NK, int* dst_rank, int64_t* dst_pos, int64_t* home_pos,
             int* off_local, int* tags, unsigned long long* dropped, cudaStream_t stream);
void ep_resolve(const int* tags, const PeerPtrs& in_bufs, const PeerPtrs& out_bufs, int64_t cap, int64_t row_bytes,
                unsigned long long* row_src, unsigned long long* row_dst, float* scale, cudaStream_t stream);

// ---- comm/tp_gemm.cu: tensor-parallel GEMMs fused with their collective (bf16; T tokens over `world` ranks)
// C[T,N] = gather(shards)[T,K] * op(B); the kernel itself fills `gathered` from the ranks' shards (peer memory)
// while it computes; `ready` is int[T/128], zeroed by the caller before the call, ready_target = 128*K*2/8192.
void tp_gemm_ag(const PeerPtrs& shards, void* gathered, const void* B, void* C, int T, int N, int K, int rank, int world,
                bool b_mn_major, int* ready, int ready_target, int* status, int num_sms, cudaStream_t stream);
// partial[T,N] = A[T,K] * op(B), rows of rank i stored into staging_slots.p[i] ([T/world, N], peer memory).
void tp_gemm_rs(const void* A, const void* B, const PeerPtrs& staging_slots, int T, int N, int K, int rank, int world,
                bool b_mn_major, int* status, int num_sms, cudaStream_t stream);
void tp_reduce_slots(const void* staging, void* y, int slots, int64_t slot_elems, cudaStream_t stream);
// C[T,N] = A[T,K] * W[K,N] with W sharded over ranks by rows of K (w_shards: each rank's [K/world, N] shard in
// symmetric memory); the kernel assembles W in `w_full` while it computes.  ready: int[K/64], zeroed by the caller.
void fsdp_gemm_agw(const void* A, const PeerPtrs& w_shards, void* w_full, void* C, int T, int N, int K, int rank,
                   int world, int* ready, int* status, int num_sms, cudaStream_t stream);

// ---- gemm/dense_bf16_2cta.cu: the same product on CTA pairs (tcgen05 cta_group::2, 256x256 tiles), same operand rules
void gemm_bf16_pair(const void* A, const void* B, void* C, int M, int N, int K, int64_t lda, int64_t ldb, int64_t ldc,
                    bool a_mn_major, bool b_mn_major, bool out_f32, bool accumulate, int* status, int num_sms,
                    cudaStream_t stream);
// Gated-MLP front half in one pair GEMM: GU[:, :I] = X Wg, GU[:, I:] = X Wu, H = act(gate) * up  (I % 128 == 0)
void gemm_gate_up_act_pair(const void* X, const void* Wg, const void* Wu, void* GU, void* H, int T, int I, int K,
                           int64_t ldx, int act, int* status, int num_sms, cudaStream_t stream);
// dGU[:, :I] = (dY Wd^T) * U * act'(G), dGU[:, I:] = (dY Wd^T) * act(G)  with G | U the halves of GU  (I % 256 == 0)
void gemm_gated_bwd_pair(const void* dY, const void* Wd, const void* GU, void* dGU, int T, int I, int D, int64_t ldy,
                         int act, int* status, int num_sms, cudaStream_t stream);

// ---- gemm/mxfp8_gemm.cu: block-scaled FP8 (e4m3 elements, one UE8M0 scale per 32 elements along K)
int64_t mxfp8_sf_bytes(int rows, int K, bool b_operand);
void mxfp8_quantize(const void* x_bf16, int R, int C, void* q, void* sf, bool q_b_operand, void* qt, void* sft,
                    bool qt_b_operand, cudaStream_t stream);
void gemm_mxfp8(const void* A, const void* sfa, const void* B, const void* sfb, void* C, int M, int N, int K, int* status,
                int num_sms, cudaStream_t stream);
// Stack of expert matrices w [E, R, C] bf16 -> q [E, R, C] (groups along C) and / or qt [E, C, R] (groups along R),
// each matrix with its own B-operand scale tiling (E * mxfp8_sf_bytes(...) bytes per scale buffer).
void mxfp8_quantize_stack(const void* w, int E, int R, int C, void* q, void* sf, void* qt, void* sft, cudaStream_t stream);
// Block-scaled grouped product: rows of X grouped by expert at 128-aligned `offsets`; B = [E, N, K] e4m3.
void grouped_gemm_mxfp8(const void* X, const void* sfa, const void* B, const void* sfb, void* Y, const int* offsets, int E,
                        int M_cap, int N, int K, int* status, int num_sms, cudaStream_t stream);

// ---- gemm/fp8_gemm.cu: per-tensor-scaled FP8 GEMM (both operands K-major) and its quantisation kernels
void fp8_amax(const void* x_bf16, int64_t n, float* amax, cudaStream_t stream);
// scale[0] = (e5m2 ? 57344 : 448) / amax[0]; q [R,C] and / or qt [C,R] (either may be null) = fp8(x * scale)
void fp8_quantize(const void* x_bf16, const float* amax, float* scale, void* q, void* qt, int R, int C, bool e5m2,
                  cudaStream_t stream);
// C[M,N] bf16 = A[M,K] * B[N,K]^T / (scale_a[0] * scale_b[0])
void gemm_fp8(const void* A, const void* B, void* C, int M, int N, int K, bool a_e5m2, bool b_e5m2, const float* scale_a,
              const float* scale_b, int* status, int num_sms, cudaStream_t stream);

// ---- elementwise/conv1d.cu: depth-wise causal conv1d + SiLU (x, y, dy, dx: bf16 [B,S,C]; w: bf16 [C,K]; dw: fp32 [C,K], added to)
void conv1d_silu_fwd(const void* x, const void* w, void* y, int B, int S, int C, int K, cudaStream_t stream);
void conv1d_silu_bwd(const void* x, const void* w, const void* dy, void* dx, float* dw, int B, int S, int C, int K,
                     cudaStream_t stream);

// ---- gdn/gdn_scan.cu: inter-chunk state recurrence of the chunked Gated Delta Rule (fp32, chunk length 64).
// Per (batch*head, chunk): W, QG, KD [64, dk]; U, O, dO, dU [64, dv]; M [64, 64]; GL scalar; Sstart [dk, dv].
bool gdn_scan_supported(int dk, int dv);
void gdn_scan_fwd(const float* W, const float* U, const float* QG, const float* M, const float* KD, const float* GL,
                  float* O, float* Sstart, int BH, int C, int dk, int dv, cudaStream_t stream);
void gdn_scan_bwd(const float* W, const float* U, const float* QG, const float* M, const float* KD, const float* GL,
                  const float* Sstart, const float* dO, float* dW, float* dU, float* dQG, float* dM, float* dKD,
                  float* dGL, int BH, int C, int dk, int dv, cudaStream_t stream);

// ---- gdn/gdn_prep.cu: chunk-parallel stage of the chunked Gated Delta Rule (fp32, chunk length 64): from raw
// q, k [B,H,S,dk], v [B,H,S,dv], beta, g [B,H,S] (any batch / head / token strides, unit inner stride, 16-byte aligned
// rows) to the scan operands W, QG, KD [B*H, C, 64, dk], U [B*H, C, 64, dv], M, T [B*H, C, 64, 64], GL [B*H, C] with
// C = ceil(S / 64); the backward takes the operand gradients to dq, dk [B,H,S,dk], dv [B,H,S,dv], dbeta, dg [B,H,S].
struct GdnStrided {
  const float* p;
  int64_t sb, sh, ss;  // element strides of the batch, head and token axes
};
bool gdn_prep_supported(int dk, int dv);
void gdn_prep_fwd(const GdnStrided& q, const GdnStrided& k, const GdnStrided& v, const GdnStrided& beta, const GdnStrided& g,
                  float* W, float* U, float* QG, float* M, float* KD, float* GL, float* T, int B, int H, int S, int dk, int dv,
                  cudaStream_t stream);
void gdn_prep_bwd(const GdnStrided& q, const GdnStrided& k, const GdnStrided& v, const GdnStrided& beta, const GdnStrided& g,
                  const float* T, const float* dW, const float* dU, const float* dQG, const float* dM, const float* dKD,
                  const float* dGL, float* dq, float* dk, float* dv_, float* dbeta, float* dg, int B, int H, int S, int dk_dim,
                  int dv, cudaStream_t stream);

// ---- moe/route.cu
void router_sigmoid_group(const void* logits, bool logits_bf16, const float* bias, float* scores, int64_t* topk_idx,
                          float* topk_w, int N, int E, int top_k, int n_group, int topk_group, bool norm, float scaling,
                          cudaStream_t stream);
void router_softmax_topk(const void* logits, bool logits_bf16, float* probs, int64_t* topk_idx, float* topk_w, int N,
                         int E, int top_k, bool norm, float scaling, cudaStream_t stream);
void router_bwd(bool softmax, const float* scores, const int64_t* topk_idx, const float* dw, const float* dscores,
                float* dlogits, int N, int E, int top_k, bool norm, float scaling, cudaStream_t stream);
int moe_sort_chunks(int M);
// experts: int64[M] expert of every flat (token, slot) entry; chunk_counts: int[moe_sort_chunks(M) * E] scratch;
// sizes int64[E]; off_p int[E+1] (128-padded); pos int64[M]; src int[cap] (entry at each padded row, -1 = padding).
void moe_sort(const int64_t* experts, int M, int E, int64_t cap, int* chunk_counts, int64_t* sizes, int* off_p,
              int64_t* pos, int* src, cudaStream_t stream);
void moe_gather_rows(const void* x, const int* src, const float* w, void* rows, int64_t cap, int K, int D,
                     int64_t entries, cudaStream_t stream);
void moe_combine_rows(const void* y, const int64_t* pos, const float* w, void* out, const void* g, float* dw, int N,
                      int K, int D, int64_t y_rows, cudaStream_t stream);

// ---- attention/flash_fwd.cu, flash_bwd.cu
struct AttnParams {
  const void* q; const void* k; const void* v; void* o; float* lse;
  const void* dout; void* dq_accum; void* dq_out; void* dk; void* dv; float* delta;
  int B, S, H, Hkv, dh;
  int dv_dim = 0;  // value / output head dim when it differs from the query / key head dim `dh` (0: same)
  // elements between consecutive tokens of each tensor (heads are packed: head h starts at h*dh)
  int64_t q_row_stride, k_row_stride, v_row_stride, o_row_stride;
  int64_t do_row_stride, dq_row_stride, dk_row_stride, dv_row_stride;
  float scale; float softcap; int window;  // window <= 0: none
  int causal;
  int* status;
};
void flash_attn_fwd(const AttnParams& p, int num_sms, cudaStream_t stream);
void flash_attn_bwd(const AttnParams& p, int num_sms, cudaStream_t stream);
// main kernel of the head_dim-64 backward with pipelined 64-query steps (attention/flash_bwd_pipe64.cu); called by
// flash_attn_bwd between its pre- and post-pass
void flash_bwd_pipe64_main(const AttnParams& p, cudaStream_t stream);

}  // namespace mt
