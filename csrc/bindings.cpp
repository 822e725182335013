// Python bindings (torch tensors in, raw launchers out).  Shape/dtype/alignment checks live here so the
// kernels can assume them.  Every function enqueues on the current CUDA stream of the tensors' device.
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include "api.h"
#include "common/bounds.cuh"

namespace {

cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

int sm_count() {
  static int n = 0;
  if (!n) n = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  return n;
}

void check_bf16_2d(const torch::Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
  TORCH_CHECK(t.scalar_type() == torch::kBFloat16, name, " must be bf16");
  TORCH_CHECK(t.dim() == 2, name, " must be 2-D");
  TORCH_CHECK(t.stride(1) == 1, name, " must have unit inner stride");
  TORCH_CHECK(t.stride(0) % 8 == 0, name, " row pitch must be a multiple of 8 elements (16 bytes)");
  TORCH_CHECK(reinterpret_cast<uintptr_t>(t.data_ptr()) % 16 == 0, name, " must be 16-byte aligned");
}

// C[M,N] (+)= op(A) op(B).  trans_a: A is stored [K,M];  trans_b == false: B is stored [N,K] (K contiguous),
// trans_b == true: B is stored [K,N].
void gemm(const torch::Tensor& A, const torch::Tensor& B, torch::Tensor& C, bool a_is_km, bool b_is_kn,
          bool accumulate, torch::Tensor& status) {
  check_bf16_2d(A, "A");
  check_bf16_2d(B, "B");
  TORCH_CHECK(C.is_cuda() && C.dim() == 2 && C.stride(1) == 1, "C must be 2-D CUDA with unit inner stride");
  const bool out_f32 = C.scalar_type() == torch::kFloat32;
  TORCH_CHECK(out_f32 || C.scalar_type() == torch::kBFloat16, "C must be bf16 or fp32");
  TORCH_CHECK((C.stride(0) * (out_f32 ? 4 : 2)) % 16 == 0, "C row pitch must be a multiple of 16 bytes");
  const int64_t M = a_is_km ? A.size(1) : A.size(0);
  const int64_t K = a_is_km ? A.size(0) : A.size(1);
  const int64_t N = b_is_kn ? B.size(1) : B.size(0);
  const int64_t Kb = b_is_kn ? B.size(0) : B.size(1);
  TORCH_CHECK(K == Kb, "contraction sizes differ: ", K, " vs ", Kb);
  TORCH_CHECK(C.size(0) == M && C.size(1) == N, "C has the wrong shape");
  c10::cuda::CUDAGuard guard(A.device());
  mt::gemm_bf16(A.data_ptr(), B.data_ptr(), C.data_ptr(), (int)M, (int)N, (int)K, A.stride(0), B.stride(0),
                C.stride(0), a_is_km, b_is_kn, out_f32, accumulate, status.data_ptr<int>(), sm_count(), cur_stream());
}

void rmsnorm_fwd(const torch::Tensor& x, const c10::optional<torch::Tensor>& residual, const torch::Tensor& w,
                 torch::Tensor& y, const c10::optional<torch::Tensor>& residual_out, torch::Tensor& rstd, double eps) {
  const int dim = (int)x.size(-1);
  TORCH_CHECK(dim % 8 == 0, "rmsnorm dim must be a multiple of 8");
  TORCH_CHECK(x.is_contiguous() && y.is_contiguous() && x.scalar_type() == torch::kBFloat16);
  TORCH_CHECK(w.scalar_type() == torch::kFloat32 && w.numel() == dim);
  const int64_t rows = x.numel() / dim;
  c10::cuda::CUDAGuard guard(x.device());
  mt::rmsnorm_fwd(x.data_ptr(), residual ? residual->data_ptr() : nullptr, w.data_ptr<float>(), y.data_ptr(),
                  residual_out ? residual_out->data_ptr() : nullptr, rstd.data_ptr<float>(), rows, dim, (float)eps,
                  cur_stream());
}

void rmsnorm_bwd(const torch::Tensor& x, const torch::Tensor& w, const torch::Tensor& rstd, const torch::Tensor& dy,
                 const c10::optional<torch::Tensor>& dres, torch::Tensor& dx, torch::Tensor& dw_partial,
                 torch::Tensor& dw, bool accumulate) {
  const int dim = (int)x.size(-1);
  const int64_t rows = x.numel() / dim;
  TORCH_CHECK(dy.is_contiguous() && x.is_contiguous() && dx.is_contiguous());
  TORCH_CHECK(dw_partial.dim() == 2 && dw_partial.size(1) == dim && dw_partial.scalar_type() == torch::kFloat32);
  const int parts = (int)dw_partial.size(0);
  c10::cuda::CUDAGuard guard(x.device());
  mt::rmsnorm_bwd(x.data_ptr(), w.data_ptr<float>(), rstd.data_ptr<float>(), dy.data_ptr(),
                  dres ? dres->data_ptr() : nullptr, dx.data_ptr(), dw_partial.data_ptr<float>(), parts, rows, dim,
                  cur_stream());
  mt::rmsnorm_bwd_reduce(dw_partial.data_ptr<float>(), parts, dim, dw.data_ptr<float>(), accumulate, cur_stream());
}

void rope(torch::Tensor& x, const torch::Tensor& cos_t, const torch::Tensor& sin_t,
          const c10::optional<torch::Tensor>& positions, int64_t seq_len, int64_t heads, int64_t head_dim,
          int64_t rot_dim, bool interleave, bool inverse) {
  // x: [tokens, row_stride] view whose first heads*head_dim columns are rotated
  TORCH_CHECK(x.dim() == 2 && x.stride(1) == 1 && x.scalar_type() == torch::kBFloat16);
  TORCH_CHECK(cos_t.scalar_type() == torch::kFloat32 && cos_t.size(1) == rot_dim / 2);
  c10::cuda::CUDAGuard guard(x.device());
  mt::rope_inplace(x.data_ptr(), cos_t.data_ptr<float>(), sin_t.data_ptr<float>(),
                   positions ? positions->data_ptr<int>() : nullptr, x.size(0), (int)seq_len, (int)heads,
                   (int)head_dim, (int)rot_dim, x.stride(0), interleave, inverse, cur_stream());
}

void rope_apply(const torch::Tensor& src, torch::Tensor& dst, const torch::Tensor& cos_t, const torch::Tensor& sin_t,
                const c10::optional<torch::Tensor>& positions, int64_t seq_len, int64_t heads, int64_t head_dim,
                int64_t rot_dim, bool inverse) {
  TORCH_CHECK(src.dim() == 2 && dst.dim() == 2 && src.stride(1) == 1 && dst.stride(1) == 1);
  TORCH_CHECK(src.scalar_type() == torch::kBFloat16 && dst.scalar_type() == torch::kBFloat16);
  TORCH_CHECK(rot_dim % 16 == 0 && head_dim % 8 == 0 && src.stride(0) % 8 == 0 && dst.stride(0) % 8 == 0);
  TORCH_CHECK(reinterpret_cast<uintptr_t>(src.data_ptr()) % 16 == 0 && reinterpret_cast<uintptr_t>(dst.data_ptr()) % 16 == 0);
  TORCH_CHECK(cos_t.size(1) == rot_dim / 2 && cos_t.is_contiguous() && sin_t.is_contiguous());
  c10::cuda::CUDAGuard guard(src.device());
  mt::rope_apply(src.data_ptr(), dst.data_ptr(), cos_t.data_ptr<float>(), sin_t.data_ptr<float>(),
                 positions ? positions->data_ptr<int>() : nullptr, src.size(0), (int)seq_len, (int)heads,
                 (int)head_dim, (int)rot_dim, src.stride(0), dst.stride(0), inverse, cur_stream());
}

void gated_act_fwd(const torch::Tensor& gate_up, torch::Tensor& out, int64_t act) {
  TORCH_CHECK(gate_up.is_contiguous() && out.is_contiguous());
  const int inter = (int)out.size(-1);
  TORCH_CHECK(gate_up.size(-1) == 2 * inter && inter % 8 == 0);
  c10::cuda::CUDAGuard guard(out.device());
  mt::gated_act_fwd(gate_up.data_ptr(), out.data_ptr(), out.numel() / inter, inter, (int)act, cur_stream());
}

void gated_act_bwd(const torch::Tensor& gate_up, const torch::Tensor& dout, torch::Tensor& dgate_up, int64_t act) {
  TORCH_CHECK(gate_up.is_contiguous() && dout.is_contiguous() && dgate_up.is_contiguous());
  const int inter = (int)dout.size(-1);
  c10::cuda::CUDAGuard guard(dout.device());
  mt::gated_act_bwd(gate_up.data_ptr(), dout.data_ptr(), dgate_up.data_ptr(), dout.numel() / inter, inter, (int)act,
                    cur_stream());
}

static void check_gate_rows(const torch::Tensor& t, const char* what) {
  TORCH_CHECK(t.dim() == 2 && t.scalar_type() == torch::kBFloat16 && t.stride(1) == 1 && t.stride(0) % 8 == 0 &&
                  t.size(1) % 8 == 0 && reinterpret_cast<uintptr_t>(t.data_ptr()) % 16 == 0,
              what, ": want bf16 rows of a multiple of 8 elements at a 16-byte-aligned pitch");
}

// out[rows, dim] = x * f(gate); x and gate are 2-D views whose rows may be strided (mode 0 sigmoid, 1 silu)
torch::Tensor gate_mul_fwd(const torch::Tensor& x, const torch::Tensor& gate, int64_t mode) {
  check_gate_rows(x, "x");
  check_gate_rows(gate, "gate");
  TORCH_CHECK(x.sizes() == gate.sizes());
  c10::cuda::CUDAGuard guard(x.device());
  auto out = torch::empty({x.size(0), x.size(1)}, x.options());
  mt::gate_mul_fwd(x.data_ptr(), gate.data_ptr(), out.data_ptr(), x.size(0), (int)x.size(1), x.stride(0), gate.stride(0),
                   (int)mode, cur_stream());
  return out;
}

// -> (dx, dgate), both contiguous [rows, dim]
std::vector<torch::Tensor> gate_mul_bwd(const torch::Tensor& x, const torch::Tensor& gate, const torch::Tensor& dout,
                                        int64_t mode) {
  check_gate_rows(x, "x");
  check_gate_rows(gate, "gate");
  TORCH_CHECK(dout.is_contiguous() && dout.scalar_type() == torch::kBFloat16 && dout.sizes() == x.sizes());
  c10::cuda::CUDAGuard guard(x.device());
  auto dx = torch::empty({x.size(0), x.size(1)}, x.options());
  auto dg = torch::empty({x.size(0), x.size(1)}, x.options());
  mt::gate_mul_bwd(x.data_ptr(), gate.data_ptr(), dout.data_ptr(), dx.data_ptr(), dg.data_ptr(), x.size(0), (int)x.size(1),
                   x.stride(0), gate.stride(0), (int)mode, cur_stream());
  return {dx, dg};
}

void cross_entropy(torch::Tensor& logits, const torch::Tensor& targets, torch::Tensor& loss,
                   const c10::optional<torch::Tensor>& zloss, const c10::optional<torch::Tensor>& lse,
                   double label_smoothing, double z_weight, double softcap, double grad_scale, bool write_grad) {
  TORCH_CHECK(logits.dim() == 2 && logits.stride(1) == 1 && logits.scalar_type() == torch::kBFloat16);
  TORCH_CHECK(logits.stride(0) % 8 == 0, "logits row pitch must be a multiple of 8");
  TORCH_CHECK(targets.scalar_type() == torch::kInt64 && targets.is_contiguous());
  c10::cuda::CUDAGuard guard(logits.device());
  mt::cross_entropy_fwd_bwd(logits.data_ptr(), targets.data_ptr<int64_t>(), loss.data_ptr<float>(),
                            zloss ? zloss->data_ptr<float>() : nullptr, lse ? lse->data_ptr<float>() : nullptr,
                            logits.size(0), (int)logits.size(1), logits.stride(0), (float)label_smoothing,
                            (float)z_weight, (float)softcap, (float)grad_scale, write_grad, cur_stream());
}

void threefry_randint(torch::Tensor& out, int64_t a0, int64_t a1, int64_t b0, int64_t b1, int64_t start, int64_t span) {
  TORCH_CHECK(out.is_cuda() && out.is_contiguous() && out.scalar_type() == torch::kInt64);
  TORCH_CHECK(span > 0 && span <= 0xFFFFFFFFll && start >= 0);
  c10::cuda::CUDAGuard guard(out.device());
  mt::threefry_randint(out.data_ptr<int64_t>(), out.numel(), (uint32_t)a0, (uint32_t)a1, (uint32_t)b0, (uint32_t)b1,
                       (uint64_t)start, (uint32_t)span, cur_stream());
}

void embedding_fwd(const torch::Tensor& table, const torch::Tensor& ids, torch::Tensor& out, double scale) {
  TORCH_CHECK(table.is_contiguous() && out.is_contiguous() && ids.is_contiguous());
  TORCH_CHECK(table.scalar_type() == torch::kBFloat16 && ids.scalar_type() == torch::kInt64);
  const int dim = (int)table.size(1);
  TORCH_CHECK(dim % 8 == 0);
  c10::cuda::CUDAGuard guard(table.device());
  mt::embedding_fwd(table.data_ptr(), ids.data_ptr<int64_t>(), out.data_ptr(), ids.numel(), dim, (float)scale,
                    table.size(0), cur_stream());
}

void embedding_bwd(const torch::Tensor& dout, const torch::Tensor& ids, torch::Tensor& dtable, double scale) {
  TORCH_CHECK(dout.is_contiguous() && ids.is_contiguous() && dtable.is_contiguous());
  TORCH_CHECK(dtable.scalar_type() == torch::kFloat32);
  const int dim = (int)dtable.size(1);
  c10::cuda::CUDAGuard guard(dout.device());
  mt::embedding_bwd(dout.data_ptr(), ids.data_ptr<int64_t>(), dtable.data_ptr<float>(), ids.numel(), dim,
                    (float)scale, dtable.size(0), cur_stream());
}

void adamw_step(torch::Tensor& master, torch::Tensor& m, torch::Tensor& v, const torch::Tensor& grad,
                const c10::optional<torch::Tensor>& param_bf16, double lr, double b1, double b2, double eps, double wd,
                double bc1, double bc2, double grad_scale, const c10::optional<torch::Tensor>& clip_coef) {
  TORCH_CHECK(master.is_contiguous() && m.is_contiguous() && v.is_contiguous() && grad.is_contiguous());
  const bool gf32 = grad.scalar_type() == torch::kFloat32;
  c10::cuda::CUDAGuard guard(master.device());
  mt::adamw_step(master.data_ptr<float>(), m.data_ptr<float>(), v.data_ptr<float>(), grad.data_ptr(), gf32,
                 param_bf16 ? param_bf16->data_ptr() : nullptr, master.numel(), (float)lr, (float)b1, (float)b2,
                 (float)eps, (float)wd, (float)bc1, (float)bc2, (float)grad_scale,
                 clip_coef ? clip_coef->data_ptr<float>() : nullptr, cur_stream());
}

void sumsq(const torch::Tensor& x, torch::Tensor& out) {
  TORCH_CHECK(x.is_contiguous() && out.scalar_type() == torch::kFloat32);
  c10::cuda::CUDAGuard guard(x.device());
  mt::sumsq(x.data_ptr(), x.scalar_type() == torch::kFloat32, x.numel(), out.data_ptr<float>(), cur_stream());
}

mt::AttnParams attn_params(const torch::Tensor& q, const torch::Tensor& k, const torch::Tensor& v, double scale,
                           bool causal, int64_t window, double softcap, torch::Tensor& status) {
  TORCH_CHECK(q.dim() == 4 && k.dim() == 4 && v.dim() == 4, "q/k/v must be [B,S,H,d]");
  for (const auto* t : {&q, &k, &v}) {
    TORCH_CHECK(t->is_cuda() && t->scalar_type() == torch::kBFloat16, "attention tensors must be CUDA bf16");
    TORCH_CHECK(t->stride(3) == 1 && t->stride(2) == t->size(3), "heads must be packed along the row");
    TORCH_CHECK(t->stride(0) == t->stride(1) * t->size(1), "batch must be contiguous in tokens");
    TORCH_CHECK(t->stride(1) % 8 == 0 && reinterpret_cast<uintptr_t>(t->data_ptr()) % 16 == 0, "16-byte alignment");
  }
  mt::AttnParams p{};
  p.q = q.data_ptr(); p.k = k.data_ptr(); p.v = v.data_ptr();
  p.B = (int)q.size(0); p.S = (int)q.size(1); p.H = (int)q.size(2); p.Hkv = (int)k.size(2); p.dh = (int)q.size(3);
  p.dv_dim = (int)v.size(3);
  TORCH_CHECK(k.size(3) == q.size(3), "q and k head dims differ");
  p.q_row_stride = q.stride(1); p.k_row_stride = k.stride(1); p.v_row_stride = v.stride(1);
  p.scale = (float)scale; p.softcap = (float)softcap; p.window = (int)window; p.causal = causal ? 1 : 0;
  p.status = status.data_ptr<int>();
  return p;
}

void flash_fwd(const torch::Tensor& q, const torch::Tensor& k, const torch::Tensor& v, torch::Tensor& o,
               torch::Tensor& lse, double scale, bool causal, int64_t window, double softcap, torch::Tensor& status) {
  mt::AttnParams p = attn_params(q, k, v, scale, causal, window, softcap, status);
  TORCH_CHECK(o.is_contiguous() && lse.is_contiguous() && lse.scalar_type() == torch::kFloat32);
  p.o = o.data_ptr(); p.o_row_stride = o.stride(1); p.lse = lse.data_ptr<float>();
  c10::cuda::CUDAGuard guard(q.device());
  mt::flash_attn_fwd(p, sm_count(), cur_stream());
}

void flash_bwd(const torch::Tensor& q, const torch::Tensor& k, const torch::Tensor& v, const torch::Tensor& o,
               const torch::Tensor& lse, const torch::Tensor& dout, torch::Tensor& dq, torch::Tensor& dk,
               torch::Tensor& dv, torch::Tensor& dq_accum, torch::Tensor& delta, double scale, bool causal,
               int64_t window, double softcap, torch::Tensor& status) {
  mt::AttnParams p = attn_params(q, k, v, scale, causal, window, softcap, status);
  TORCH_CHECK(o.is_contiguous() && dout.is_contiguous() && dq.is_contiguous() && dk.is_contiguous() && dv.is_contiguous());
  TORCH_CHECK(dq_accum.scalar_type() == torch::kFloat32 && dq_accum.numel() == q.size(0) * q.size(1) * q.size(2) * q.size(3) &&
              dq_accum.is_contiguous());
  TORCH_CHECK(delta.scalar_type() == torch::kFloat32 && delta.numel() == lse.numel());
  p.o = const_cast<void*>(o.data_ptr()); p.o_row_stride = o.stride(1);
  p.lse = const_cast<float*>(lse.data_ptr<float>());
  p.dout = dout.data_ptr(); p.do_row_stride = dout.stride(1);
  p.dq_accum = dq_accum.data_ptr(); p.dq_out = dq.data_ptr(); p.dq_row_stride = dq.stride(1);
  p.dk = dk.data_ptr(); p.dk_row_stride = dk.stride(1);
  p.dv = dv.data_ptr(); p.dv_row_stride = dv.stride(1);
  p.delta = delta.data_ptr<float>();
  c10::cuda::CUDAGuard guard(q.device());
  mt::flash_attn_bwd(p, sm_count(), cur_stream());
}

mt::PeerPtrs to_peers(const std::vector<int64_t>& ptrs) {
  TORCH_CHECK((int)ptrs.size() <= mt::kMaxPeers, "at most ", mt::kMaxPeers, " peers");
  mt::PeerPtrs p{};
  for (size_t i = 0; i < ptrs.size(); ++i) p.p[i] = reinterpret_cast<void*>(ptrs[i]);
  return p;
}

void symm_barrier(const std::vector<int64_t>& flag_ptrs, int64_t rank, int64_t seq, torch::Tensor& status) {
  c10::cuda::CUDAGuard guard(status.device());
  mt::symm_barrier(to_peers(flag_ptrs), (int)rank, (int)flag_ptrs.size(), (int)seq, status.data_ptr<int>(), cur_stream());
}

void grad_pull_reduce(const std::vector<int64_t>& grad_ptrs, int64_t rank, int64_t lo, torch::Tensor& out,
                      torch::Tensor& sumsq) {
  TORCH_CHECK(out.scalar_type() == torch::kFloat32 && out.is_contiguous() && out.numel() % 4 == 0 && lo % 4 == 0);
  c10::cuda::CUDAGuard guard(out.device());
  mt::grad_pull_reduce(to_peers(grad_ptrs), (int)rank, (int)grad_ptrs.size(), lo, out.numel(), out.data_ptr<float>(),
                       sumsq.data_ptr<float>(), cur_stream());
}

void grad_pull_bucket(const std::vector<int64_t>& grad_ptrs, const std::vector<int64_t>& flag_ptrs, int64_t rank,
                      int64_t bucket, int64_t seq, int64_t lo, torch::Tensor& out, bool accumulate, bool clear,
                      bool handshake, int64_t blocks, torch::Tensor& status) {
  TORCH_CHECK(out.scalar_type() == torch::kFloat32 && out.is_contiguous() && out.numel() % 4 == 0 && lo % 4 == 0);
  TORCH_CHECK(grad_ptrs.size() == flag_ptrs.size() && bucket >= 0 && bucket < mt::kBucketSlots);
  c10::cuda::CUDAGuard guard(out.device());
  mt::grad_pull_bucket(to_peers(grad_ptrs), to_peers(flag_ptrs), (int)rank, (int)grad_ptrs.size(), (int)bucket, (int)seq,
                       lo, out.numel(), out.data_ptr<float>(), accumulate, clear, handshake, (int)blocks,
                       status.data_ptr<int>(), cur_stream());
}

void bucket_ready(const std::vector<int64_t>& flag_ptrs, int64_t rank, int64_t bucket, int64_t seq, torch::Tensor& status) {
  TORCH_CHECK(bucket >= 0 && bucket < mt::kBucketSlots);
  c10::cuda::CUDAGuard guard(status.device());
  mt::bucket_ready(to_peers(flag_ptrs), (int)rank, (int)flag_ptrs.size(), (int)bucket, (int)seq, status.data_ptr<int>(),
                   cur_stream());
}

int64_t bucket_flag_slots() { return mt::kBucketSlots; }

// dst (flat, world * n elements) <- elements [lo + r * rank_stride, + n) of rank r's buffer, rank by rank
void peer_gather(const std::vector<int64_t>& shard_ptrs, int64_t lo, int64_t rank_stride, int64_t n, torch::Tensor& dst,
                 int64_t blocks) {
  const int64_t es = dst.element_size();
  TORCH_CHECK(dst.is_cuda() && dst.is_contiguous() && dst.numel() == n * (int64_t)shard_ptrs.size());
  TORCH_CHECK((lo * es) % 16 == 0 && (n * es) % 16 == 0 && (rank_stride * es) % 16 == 0 &&
              reinterpret_cast<uintptr_t>(dst.data_ptr()) % 16 == 0);
  c10::cuda::CUDAGuard guard(dst.device());
  mt::peer_gather(to_peers(shard_ptrs), (int)shard_ptrs.size(), lo * es, rank_stride * es, n * es, dst.data_ptr(),
                  (int)blocks, cur_stream());
}

void adamw_publish(torch::Tensor& master, torch::Tensor& m, torch::Tensor& v, const torch::Tensor& grad,
                   const std::vector<int64_t>& param_ptrs, int64_t lo, double lr, double b1, double b2, double eps,
                   double wd, double bc1, double bc2, double grad_scale, const c10::optional<torch::Tensor>& clip_coef) {
  TORCH_CHECK(master.numel() % 8 == 0 && lo % 8 == 0 && grad.scalar_type() == torch::kFloat32);
  c10::cuda::CUDAGuard guard(master.device());
  mt::adamw_publish(master.data_ptr<float>(), m.data_ptr<float>(), v.data_ptr<float>(), grad.data_ptr<float>(),
                    to_peers(param_ptrs), (int)param_ptrs.size(), lo, master.numel(), (float)lr, (float)b1, (float)b2,
                    (float)eps, (float)wd, (float)bc1, (float)bc2, (float)grad_scale,
                    clip_coef ? clip_coef->data_ptr<float>() : nullptr, cur_stream());
}

void grouped_gemm(const torch::Tensor& x, const torch::Tensor& w, torch::Tensor& y, const torch::Tensor& offsets,
                  bool w_is_ekn, torch::Tensor& status) {
  // x [M_cap, K] bf16, rows grouped by expert at 128-aligned offsets ; w [E, K, N] (w_is_ekn) or [E, N, K]
  check_bf16_2d(x, "x");
  TORCH_CHECK(w.dim() == 3 && w.is_contiguous() && w.scalar_type() == torch::kBFloat16, "w must be contiguous bf16 [E,.,.]");
  TORCH_CHECK(y.is_contiguous() && y.scalar_type() == torch::kBFloat16 && x.is_contiguous());
  TORCH_CHECK(offsets.scalar_type() == torch::kInt32 && offsets.is_contiguous() && offsets.numel() == w.size(0) + 1);
  const int64_t K = x.size(1);
  const int64_t N = w_is_ekn ? w.size(2) : w.size(1);
  TORCH_CHECK((w_is_ekn ? w.size(1) : w.size(2)) == K, "contraction sizes differ");
  TORCH_CHECK(y.size(0) == x.size(0) && y.size(1) == N && x.size(0) % 128 == 0 && K % 8 == 0 && N % 8 == 0);
  c10::cuda::CUDAGuard guard(x.device());
  mt::grouped_gemm_bf16(x.data_ptr(), w.data_ptr(), y.data_ptr(), offsets.data_ptr<int>(), (int)w.size(0),
                        (int)x.size(0), (int)N, (int)K, w_is_ekn, status.data_ptr<int>(), sm_count(), cur_stream());
}

// Expert GEMM fused with a row scatter: output row r is written to the byte address row_dst[r] (int64; 0 drops the
// row), which may lie in a peer GPU's symmetric buffer.  Rows are N bf16 wide.
void grouped_gemm_scatter(const torch::Tensor& x, const torch::Tensor& w, const torch::Tensor& row_dst,
                          const torch::Tensor& offsets, bool w_is_ekn, torch::Tensor& status) {
  check_bf16_2d(x, "x");
  TORCH_CHECK(w.dim() == 3 && w.is_contiguous() && w.scalar_type() == torch::kBFloat16 && x.is_contiguous());
  TORCH_CHECK(row_dst.scalar_type() == torch::kInt64 && row_dst.is_contiguous() && row_dst.numel() == x.size(0));
  TORCH_CHECK(offsets.scalar_type() == torch::kInt32 && offsets.is_contiguous() && offsets.numel() == w.size(0) + 1);
  const int64_t K = x.size(1);
  const int64_t N = w_is_ekn ? w.size(2) : w.size(1);
  TORCH_CHECK((w_is_ekn ? w.size(1) : w.size(2)) == K && x.size(0) % 128 == 0 && K % 8 == 0 && N % 8 == 0 && N > 128);
  c10::cuda::CUDAGuard guard(x.device());
  mt::grouped_gemm_scatter_bf16_pair(x.data_ptr(), w.data_ptr(),
                                     reinterpret_cast<const unsigned long long*>(row_dst.data_ptr<int64_t>()),
                                     offsets.data_ptr<int>(), (int)w.size(0), (int)x.size(0), (int)N, (int)K, w_is_ekn,
                                     status.data_ptr<int>(), sm_count(), cur_stream());
}

void grouped_wgrad(const torch::Tensor& x, const torch::Tensor& g, torch::Tensor& dw, const torch::Tensor& offsets,
                   bool accumulate, torch::Tensor& status) {
  check_bf16_2d(x, "x");
  check_bf16_2d(g, "g");
  TORCH_CHECK(x.is_contiguous() && g.is_contiguous() && dw.is_contiguous() && dw.dim() == 3);
  const bool f32 = dw.scalar_type() == torch::kFloat32;
  TORCH_CHECK(f32 || dw.scalar_type() == torch::kBFloat16);
  TORCH_CHECK(dw.size(1) == x.size(1) && dw.size(2) == g.size(1) && x.size(0) == g.size(0) && x.size(0) % 128 == 0);
  TORCH_CHECK(offsets.scalar_type() == torch::kInt32 && offsets.numel() == dw.size(0) + 1);
  c10::cuda::CUDAGuard guard(x.device());
  mt::grouped_wgrad_bf16(x.data_ptr(), g.data_ptr(), dw.data_ptr(), offsets.data_ptr<int>(), (int)dw.size(0),
                         (int)x.size(0), (int)g.size(1), (int)x.size(1), f32, accumulate, status.data_ptr<int>(),
                         sm_count(), cur_stream());
}

void ep_push_rows(const torch::Tensor& src, const torch::Tensor& dst_rank, const torch::Tensor& dst_pos,
                  const std::vector<int64_t>& buf_ptrs, int64_t cap_rows, torch::Tensor& overflow) {
  TORCH_CHECK(src.is_contiguous() && src.scalar_type() == torch::kBFloat16 && src.dim() == 2 && src.size(1) % 8 == 0);
  TORCH_CHECK(dst_rank.scalar_type() == torch::kInt32 && dst_pos.scalar_type() == torch::kInt64);
  TORCH_CHECK(dst_rank.numel() == src.size(0) && dst_pos.numel() == src.size(0));
  c10::cuda::CUDAGuard guard(src.device());
  mt::ep_push_rows(src.data_ptr(), dst_rank.data_ptr<int>(), dst_pos.data_ptr<int64_t>(), to_peers(buf_ptrs), src.size(0),
                   (int)src.size(1), cap_rows, overflow.data_ptr<int>(), cur_stream());
}

void ep_pull_rows(torch::Tensor& out, const torch::Tensor& src_rank, const torch::Tensor& src_pos,
                  const std::vector<int64_t>& buf_ptrs, int64_t cap_rows) {
  TORCH_CHECK(out.is_contiguous() && out.scalar_type() == torch::kBFloat16 && out.dim() == 2 && out.size(1) % 8 == 0);
  TORCH_CHECK(src_rank.scalar_type() == torch::kInt32 && src_pos.scalar_type() == torch::kInt64);
  c10::cuda::CUDAGuard guard(out.device());
  mt::ep_pull_rows(out.data_ptr(), src_rank.data_ptr<int>(), src_pos.data_ptr<int64_t>(), to_peers(buf_ptrs), out.size(0),
                   (int)out.size(1), cap_rows, cur_stream());
}

// out [R, D] bf16; row_src int64 [R] byte addresses (0 = zero row); row_scale fp32 [R] or an empty tensor
void ep_gather_rows(torch::Tensor& out, const torch::Tensor& row_src, const torch::Tensor& row_scale) {
  TORCH_CHECK(out.is_contiguous() && out.scalar_type() == torch::kBFloat16 && out.dim() == 2 && out.size(1) % 8 == 0);
  TORCH_CHECK(row_src.scalar_type() == torch::kInt64 && row_src.is_contiguous() && row_src.numel() == out.size(0));
  const bool scaled = row_scale.numel() > 0;
  if (scaled) TORCH_CHECK(row_scale.scalar_type() == torch::kFloat32 && row_scale.is_contiguous() && row_scale.numel() == out.size(0));
  c10::cuda::CUDAGuard guard(out.device());
  mt::ep_gather_rows(out.data_ptr(), reinterpret_cast<const unsigned long long*>(row_src.data_ptr<int64_t>()),
                     scaled ? row_scale.data_ptr<float>() : nullptr, out.size(0), (int)out.size(1), cur_stream());
}

// gu [T, 2I] <- [x wg | x wu], h [T, I] <- act(x wg) * (x wu); wg, wu [K, I] contiguous bf16
void gemm_gate_up_act(const torch::Tensor& x, const torch::Tensor& wg, const torch::Tensor& wu, torch::Tensor& gu,
                      torch::Tensor& h, int64_t act, torch::Tensor& status) {
  check_bf16_2d(x, "x");
  TORCH_CHECK(x.stride(1) == 1 && x.stride(0) % 8 == 0);
  TORCH_CHECK(wg.is_contiguous() && wu.is_contiguous() && wg.dim() == 2 && wg.sizes() == wu.sizes());
  TORCH_CHECK(wg.scalar_type() == torch::kBFloat16 && wu.scalar_type() == torch::kBFloat16);
  const int64_t T = x.size(0), K = x.size(1), I = wg.size(1);
  TORCH_CHECK(wg.size(0) == K && I % 128 == 0 && K % 8 == 0);
  TORCH_CHECK(gu.is_contiguous() && h.is_contiguous() && gu.scalar_type() == torch::kBFloat16 && h.scalar_type() == torch::kBFloat16);
  TORCH_CHECK(gu.size(0) == T && gu.size(1) == 2 * I && h.size(0) == T && h.size(1) == I);
  c10::cuda::CUDAGuard guard(x.device());
  mt::gemm_gate_up_act_pair(x.data_ptr(), wg.data_ptr(), wu.data_ptr(), gu.data_ptr(), h.data_ptr(), (int)T, (int)I, (int)K,
                            x.stride(0), (int)act, status.data_ptr<int>(), sm_count(), cur_stream());
}

// dgu [T, 2I] <- [(dy wd^T) * up * act'(gate) | (dy wd^T) * act(gate)], gate | up = halves of gu; wd [I, D]
void gemm_gated_bwd(const torch::Tensor& dy, const torch::Tensor& wd, const torch::Tensor& gu, torch::Tensor& dgu,
                    int64_t act, torch::Tensor& status) {
  check_bf16_2d(dy, "dy");
  TORCH_CHECK(dy.stride(1) == 1 && dy.stride(0) % 8 == 0);
  TORCH_CHECK(wd.is_contiguous() && wd.dim() == 2 && wd.scalar_type() == torch::kBFloat16);
  const int64_t T = dy.size(0), D = dy.size(1), I = wd.size(0);
  TORCH_CHECK(wd.size(1) == D && I % 256 == 0 && D % 8 == 0);
  TORCH_CHECK(gu.is_contiguous() && dgu.is_contiguous() && gu.scalar_type() == torch::kBFloat16 && dgu.scalar_type() == torch::kBFloat16);
  TORCH_CHECK(gu.size(0) == T && gu.size(1) == 2 * I && dgu.sizes() == gu.sizes());
  c10::cuda::CUDAGuard guard(dy.device());
  mt::gemm_gated_bwd_pair(dy.data_ptr(), wd.data_ptr(), gu.data_ptr(), dgu.data_ptr(), (int)T, (int)I, (int)D, dy.stride(0),
                          (int)act, status.data_ptr<int>(), sm_count(), cur_stream());
}

// c[M,N] = a[M,K] @ (b_kn ? b[K,N] : b[N,K]^T) on CTA pairs (bf16 in / out)
void gemm_pair(const torch::Tensor& a, const torch::Tensor& b, torch::Tensor& c, bool b_kn, torch::Tensor& status) {
  TORCH_CHECK(a.scalar_type() == torch::kBFloat16 && b.scalar_type() == torch::kBFloat16 && c.scalar_type() == torch::kBFloat16);
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && c.dim() == 2 && a.stride(1) == 1 && b.stride(1) == 1 && c.stride(1) == 1);
  const int64_t M = a.size(0), K = a.size(1), N = b_kn ? b.size(1) : b.size(0);
  TORCH_CHECK((b_kn ? b.size(0) : b.size(1)) == K && c.size(0) == M && c.size(1) == N);
  TORCH_CHECK(a.stride(0) % 8 == 0 && b.stride(0) % 8 == 0 && c.stride(0) % 8 == 0 && K % 8 == 0 && N % 8 == 0);
  c10::cuda::CUDAGuard guard(a.device());
  mt::gemm_bf16_pair(a.data_ptr(), b.data_ptr(), c.data_ptr(), (int)M, (int)N, (int)K, a.stride(0), b.stride(0), c.stride(0),
                     false, b_kn, false, false, status.data_ptr<int>(), sm_count(), cur_stream());
}

// -> (q uint8 [R,C] or undefined, qt uint8 [C,R] or undefined, scale fp32 [1])
std::vector<torch::Tensor> fp8_quantize(const torch::Tensor& x, bool e5m2, bool want_q, bool want_qt) {
  TORCH_CHECK(x.is_cuda() && x.is_contiguous() && x.dim() == 2 && x.scalar_type() == torch::kBFloat16);
  c10::cuda::CUDAGuard guard(x.device());
  auto f32 = x.options().dtype(torch::kFloat32);
  auto u8 = x.options().dtype(torch::kUInt8);
  auto amax = torch::empty({1}, f32);
  auto scale = torch::empty({1}, f32);
  torch::Tensor q, qt;
  if (want_q) q = torch::empty({x.size(0), x.size(1)}, u8);
  if (want_qt) qt = torch::empty({x.size(1), x.size(0)}, u8);
  mt::fp8_amax(x.data_ptr(), x.numel(), amax.data_ptr<float>(), cur_stream());
  mt::fp8_quantize(x.data_ptr(), amax.data_ptr<float>(), scale.data_ptr<float>(), want_q ? q.data_ptr() : nullptr,
                   want_qt ? qt.data_ptr() : nullptr, (int)x.size(0), (int)x.size(1), e5m2, cur_stream());
  return {q, qt, scale};
}

// out[M,N] bf16 = a[M,K] . b[N,K]^T / (scale_a * scale_b), 8-bit float operands
torch::Tensor gemm_fp8(const torch::Tensor& a, const torch::Tensor& b, bool a_e5m2, bool b_e5m2, const torch::Tensor& scale_a,
                       const torch::Tensor& scale_b, torch::Tensor& status) {
  TORCH_CHECK(a.is_contiguous() && b.is_contiguous() && a.scalar_type() == torch::kUInt8 && b.scalar_type() == torch::kUInt8);
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && a.size(1) == b.size(1) && a.size(1) % 16 == 0 && b.size(0) % 8 == 0);
  c10::cuda::CUDAGuard guard(a.device());
  auto out = torch::empty({a.size(0), b.size(0)}, a.options().dtype(torch::kBFloat16));
  mt::gemm_fp8(a.data_ptr(), b.data_ptr(), out.data_ptr(), (int)a.size(0), (int)b.size(0), (int)a.size(1), a_e5m2, b_e5m2,
               scale_a.data_ptr<float>(), scale_b.data_ptr<float>(), status.data_ptr<int>(), sm_count(), cur_stream());
  return out;
}

// x [R,C] bf16 -> (q [R,C], sf, qt [C,R], sft): e4m3 elements with UE8M0 scales per 32 elements along the last dim
// of q / qt; scale buffers are tiled for the GEMM's A (128-row tiles) or B (192-row tiles) operand.
std::vector<torch::Tensor> mxfp8_quantize(const torch::Tensor& x, bool want_q, bool q_b_operand, bool want_qt,
                                          bool qt_b_operand) {
  TORCH_CHECK(x.is_cuda() && x.is_contiguous() && x.dim() == 2 && x.scalar_type() == torch::kBFloat16);
  c10::cuda::CUDAGuard guard(x.device());
  auto u8 = x.options().dtype(torch::kUInt8);
  const int R = (int)x.size(0), C = (int)x.size(1);
  torch::Tensor q, sf, qt, sft;
  if (want_q) {
    q = torch::empty({R, C}, u8);
    sf = torch::zeros({mt::mxfp8_sf_bytes(R, C, q_b_operand)}, u8);
  }
  if (want_qt) {
    qt = torch::empty({C, R}, u8);
    sft = torch::zeros({mt::mxfp8_sf_bytes(C, R, qt_b_operand)}, u8);
  }
  mt::mxfp8_quantize(x.data_ptr(), R, C, want_q ? q.data_ptr() : nullptr, want_q ? sf.data_ptr() : nullptr, q_b_operand,
                     want_qt ? qt.data_ptr() : nullptr, want_qt ? sft.data_ptr() : nullptr, qt_b_operand, cur_stream());
  return {q, sf, qt, sft};
}

// out[M,N] bf16 = a[M,K] . b[N,K]^T with the block scales applied by the tensor core
torch::Tensor gemm_mxfp8(const torch::Tensor& a, const torch::Tensor& sfa, const torch::Tensor& b, const torch::Tensor& sfb,
                         torch::Tensor& status) {
  TORCH_CHECK(a.is_contiguous() && b.is_contiguous() && a.scalar_type() == torch::kUInt8 && b.scalar_type() == torch::kUInt8);
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && a.size(1) == b.size(1) && a.size(1) % 128 == 0 && b.size(0) % 8 == 0);
  TORCH_CHECK(sfa.numel() == mt::mxfp8_sf_bytes((int)a.size(0), (int)a.size(1), false), "A scales: wrong tiling");
  TORCH_CHECK(sfb.numel() == mt::mxfp8_sf_bytes((int)b.size(0), (int)b.size(1), true), "B scales: wrong tiling");
  c10::cuda::CUDAGuard guard(a.device());
  auto out = torch::empty({a.size(0), b.size(0)}, a.options().dtype(torch::kBFloat16));
  mt::gemm_mxfp8(a.data_ptr(), sfa.data_ptr(), b.data_ptr(), sfb.data_ptr(), out.data_ptr(), (int)a.size(0), (int)b.size(0),
                 (int)a.size(1), status.data_ptr<int>(), sm_count(), cur_stream());
  return out;
}

// w [E,R,C] bf16 -> (q [E,R,C], sf, qt [E,C,R], sft) with per-matrix B-operand scale tilings (expert weights)
std::vector<torch::Tensor> mxfp8_quantize_stack(const torch::Tensor& w, bool want_q, bool want_qt) {
  TORCH_CHECK(w.is_cuda() && w.is_contiguous() && w.dim() == 3 && w.scalar_type() == torch::kBFloat16);
  c10::cuda::CUDAGuard guard(w.device());
  auto u8 = w.options().dtype(torch::kUInt8);
  const int E = (int)w.size(0), R = (int)w.size(1), C = (int)w.size(2);
  torch::Tensor q, sf, qt, sft;
  if (want_q) {
    q = torch::empty({E, R, C}, u8);
    sf = torch::zeros({E * mt::mxfp8_sf_bytes(R, C, true)}, u8);
  }
  if (want_qt) {
    qt = torch::empty({E, C, R}, u8);
    sft = torch::zeros({E * mt::mxfp8_sf_bytes(C, R, true)}, u8);
  }
  mt::mxfp8_quantize_stack(w.data_ptr(), E, R, C, want_q ? q.data_ptr() : nullptr, want_q ? sf.data_ptr() : nullptr,
                           want_qt ? qt.data_ptr() : nullptr, want_qt ? sft.data_ptr() : nullptr, cur_stream());
  return {q, sf, qt, sft};
}

// y [M_cap, N] bf16 = x [M_cap, K] . b[e] [N, K]^T per expert row group, block scales applied by the tensor core
torch::Tensor grouped_gemm_mxfp8(const torch::Tensor& x, const torch::Tensor& sfx, const torch::Tensor& b,
                                 const torch::Tensor& sfb, const torch::Tensor& offsets, torch::Tensor& status) {
  TORCH_CHECK(x.is_contiguous() && b.is_contiguous() && x.scalar_type() == torch::kUInt8 && b.scalar_type() == torch::kUInt8);
  TORCH_CHECK(x.dim() == 2 && b.dim() == 3 && x.size(1) == b.size(2) && x.size(1) % 128 == 0 && b.size(1) % 8 == 0 &&
              x.size(0) % 128 == 0);
  TORCH_CHECK(offsets.scalar_type() == torch::kInt32 && offsets.is_contiguous() && offsets.numel() == b.size(0) + 1);
  TORCH_CHECK(sfx.numel() == mt::mxfp8_sf_bytes((int)x.size(0), (int)x.size(1), false), "row scales: wrong tiling");
  TORCH_CHECK(sfb.numel() == b.size(0) * mt::mxfp8_sf_bytes((int)b.size(1), (int)b.size(2), true), "expert scales: wrong tiling");
  c10::cuda::CUDAGuard guard(x.device());
  auto y = torch::empty({x.size(0), b.size(1)}, x.options().dtype(torch::kBFloat16));
  mt::grouped_gemm_mxfp8(x.data_ptr(), sfx.data_ptr(), b.data_ptr(), sfb.data_ptr(), y.data_ptr(), offsets.data_ptr<int>(),
                         (int)b.size(0), (int)x.size(0), (int)b.size(1), (int)x.size(2 - 1), status.data_ptr<int>(),
                         sm_count(), cur_stream());
  return y;
}

// W, QG, KD [BH, C, 64, dk]; U [BH, C, 64, dv]; M [BH, C, 64, 64]; GL [BH, C]  ->  (O [BH, C, 64, dv], Sstart [BH, C, dk, dv])
std::vector<torch::Tensor> gdn_scan_fwd(const torch::Tensor& W, const torch::Tensor& U, const torch::Tensor& QG,
                                        const torch::Tensor& M, const torch::Tensor& KD, const torch::Tensor& GL) {
  for (const auto* t : {&W, &U, &QG, &M, &KD, &GL})
    TORCH_CHECK(t->is_cuda() && t->is_contiguous() && t->scalar_type() == torch::kFloat32, "gdn_scan wants contiguous fp32");
  const int64_t BH = W.size(0), C = W.size(1), dk = W.size(3), dv = U.size(3);
  TORCH_CHECK(W.size(2) == 64 && M.size(2) == 64 && M.size(3) == 64 && mt::gdn_scan_supported((int)dk, (int)dv));
  c10::cuda::CUDAGuard guard(W.device());
  auto O = torch::empty_like(U);
  auto S = torch::empty({BH, C, dk, dv}, W.options());
  mt::gdn_scan_fwd(W.data_ptr<float>(), U.data_ptr<float>(), QG.data_ptr<float>(), M.data_ptr<float>(), KD.data_ptr<float>(),
                   GL.data_ptr<float>(), O.data_ptr<float>(), S.data_ptr<float>(), (int)BH, (int)C, (int)dk, (int)dv,
                   cur_stream());
  return {O, S};
}

// -> (dW, dU, dQG, dM, dKD, dGL)
std::vector<torch::Tensor> gdn_scan_bwd(const torch::Tensor& W, const torch::Tensor& U, const torch::Tensor& QG,
                                        const torch::Tensor& M, const torch::Tensor& KD, const torch::Tensor& GL,
                                        const torch::Tensor& S, const torch::Tensor& dO) {
  TORCH_CHECK(dO.is_contiguous() && dO.scalar_type() == torch::kFloat32 && S.is_contiguous());
  const int64_t BH = W.size(0), C = W.size(1), dk = W.size(3), dv = U.size(3);
  c10::cuda::CUDAGuard guard(W.device());
  auto dW = torch::zeros_like(W), dQG = torch::zeros_like(QG), dKD = torch::zeros_like(KD), dM = torch::zeros_like(M),
       dGL = torch::zeros_like(GL), dU = torch::empty_like(U);
  mt::gdn_scan_bwd(W.data_ptr<float>(), U.data_ptr<float>(), QG.data_ptr<float>(), M.data_ptr<float>(), KD.data_ptr<float>(),
                   GL.data_ptr<float>(), S.data_ptr<float>(), dO.data_ptr<float>(), dW.data_ptr<float>(), dU.data_ptr<float>(),
                   dQG.data_ptr<float>(), dM.data_ptr<float>(), dKD.data_ptr<float>(), dGL.data_ptr<float>(), (int)BH, (int)C,
                   (int)dk, (int)dv, cur_stream());
  return {dW, dU, dQG, dM, dKD, dGL};
}

static mt::GdnStrided gdn_strided(const torch::Tensor& t, bool rows) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == torch::kFloat32 && t.dim() == (rows ? 4 : 3), "gdn_prep wants fp32 [B,H,S(,d)]");
  if (rows)
    TORCH_CHECK(t.stride(3) == 1 && t.stride(0) % 4 == 0 && t.stride(1) % 4 == 0 && t.stride(2) % 4 == 0 &&
                    reinterpret_cast<uintptr_t>(t.data_ptr()) % 16 == 0,
                "gdn_prep wants unit inner stride and 16-byte aligned rows");
  return {t.data_ptr<float>(), t.stride(0), t.stride(1), t.stride(2)};
}

// q, k [B,H,S,dk], v [B,H,S,dv], beta, g [B,H,S] (strided views allowed) -> (W, U, QG, M, KD, GL, T)
std::vector<torch::Tensor> gdn_prep_fwd(const torch::Tensor& q, const torch::Tensor& k, const torch::Tensor& v,
                                        const torch::Tensor& beta, const torch::Tensor& g) {
  const int64_t B = q.size(0), H = q.size(1), S = q.size(2), dk = q.size(3), dv = v.size(3), C = (S + 63) / 64;
  TORCH_CHECK(k.sizes() == q.sizes() && v.size(0) == B && v.size(1) == H && v.size(2) == S && beta.size(2) == S &&
              g.size(2) == S && mt::gdn_prep_supported((int)dk, (int)dv));
  c10::cuda::CUDAGuard guard(q.device());
  auto o = q.options();
  auto W = torch::empty({B * H, C, 64, dk}, o), QG = torch::empty({B * H, C, 64, dk}, o), KD = torch::empty({B * H, C, 64, dk}, o);
  auto U = torch::empty({B * H, C, 64, dv}, o), M = torch::empty({B * H, C, 64, 64}, o), T = torch::empty({B * H, C, 64, 64}, o);
  auto GL = torch::empty({B * H, C}, o);
  mt::gdn_prep_fwd(gdn_strided(q, true), gdn_strided(k, true), gdn_strided(v, true), gdn_strided(beta, false),
                   gdn_strided(g, false), W.data_ptr<float>(), U.data_ptr<float>(), QG.data_ptr<float>(), M.data_ptr<float>(),
                   KD.data_ptr<float>(), GL.data_ptr<float>(), T.data_ptr<float>(), (int)B, (int)H, (int)S, (int)dk, (int)dv,
                   cur_stream());
  return {W, U, QG, M, KD, GL, T};
}

// -> (dq, dk, dv, dbeta, dg), contiguous [B,H,S,...]
std::vector<torch::Tensor> gdn_prep_bwd(const torch::Tensor& q, const torch::Tensor& k, const torch::Tensor& v,
                                        const torch::Tensor& beta, const torch::Tensor& g, const torch::Tensor& T,
                                        const torch::Tensor& dW, const torch::Tensor& dU, const torch::Tensor& dQG,
                                        const torch::Tensor& dM, const torch::Tensor& dKD, const torch::Tensor& dGL) {
  const int64_t B = q.size(0), H = q.size(1), S = q.size(2), dk = q.size(3), dv = v.size(3);
  for (const auto* t : {&T, &dW, &dU, &dQG, &dM, &dKD, &dGL})
    TORCH_CHECK(t->is_cuda() && t->is_contiguous() && t->scalar_type() == torch::kFloat32, "gdn_prep_bwd wants contiguous fp32");
  TORCH_CHECK(mt::gdn_prep_supported((int)dk, (int)dv) && dW.size(0) == B * H && dW.size(3) == dk && dU.size(3) == dv);
  c10::cuda::CUDAGuard guard(q.device());
  auto o = q.options();
  auto dq = torch::empty({B, H, S, dk}, o), dkk = torch::empty({B, H, S, dk}, o), dvv = torch::empty({B, H, S, dv}, o);
  auto dbeta = torch::empty({B, H, S}, o), dg = torch::empty({B, H, S}, o);
  mt::gdn_prep_bwd(gdn_strided(q, true), gdn_strided(k, true), gdn_strided(v, true), gdn_strided(beta, false),
                   gdn_strided(g, false), T.data_ptr<float>(), dW.data_ptr<float>(), dU.data_ptr<float>(),
                   dQG.data_ptr<float>(), dM.data_ptr<float>(), dKD.data_ptr<float>(), dGL.data_ptr<float>(),
                   dq.data_ptr<float>(), dkk.data_ptr<float>(), dvv.data_ptr<float>(), dbeta.data_ptr<float>(),
                   dg.data_ptr<float>(), (int)B, (int)H, (int)S, (int)dk, (int)dv, cur_stream());
  return {dq, dkk, dvv, dbeta, dg};
}

torch::Tensor conv1d_silu_fwd(const torch::Tensor& x, const torch::Tensor& w) {
  TORCH_CHECK(x.is_cuda() && x.is_contiguous() && x.dim() == 3 && x.scalar_type() == torch::kBFloat16);
  TORCH_CHECK(w.is_contiguous() && w.scalar_type() == torch::kBFloat16 && w.numel() % x.size(2) == 0);
  c10::cuda::CUDAGuard guard(x.device());
  auto y = torch::empty_like(x);
  mt::conv1d_silu_fwd(x.data_ptr(), w.data_ptr(), y.data_ptr(), (int)x.size(0), (int)x.size(1), (int)x.size(2),
                      (int)(w.numel() / x.size(2)), cur_stream());
  return y;
}

// -> (dx bf16 [B,S,C], dw fp32 shaped like w)
std::vector<torch::Tensor> conv1d_silu_bwd(const torch::Tensor& x, const torch::Tensor& w, const torch::Tensor& dy) {
  TORCH_CHECK(x.is_contiguous() && dy.is_contiguous() && w.is_contiguous() && dy.scalar_type() == torch::kBFloat16);
  c10::cuda::CUDAGuard guard(x.device());
  auto dx = torch::empty_like(x);
  auto dw = torch::zeros(w.sizes(), w.options().dtype(torch::kFloat32));
  mt::conv1d_silu_bwd(x.data_ptr(), w.data_ptr(), dy.data_ptr(), dx.data_ptr(), dw.data_ptr<float>(), (int)x.size(0),
                      (int)x.size(1), (int)x.size(2), (int)(w.numel() / x.size(2)), cur_stream());
  return {dx, dw};
}

// -> (topk_idx int64 [N,K], topk_w fp32 [N,K], scores fp32 [N,E]); kind 0 = sigmoid / group-limited, 1 = softmax
std::vector<torch::Tensor> moe_router(const torch::Tensor& logits, const c10::optional<torch::Tensor>& bias, int64_t kind,
                                      int64_t top_k, int64_t n_group, int64_t topk_group, bool norm, double scaling) {
  TORCH_CHECK(logits.is_cuda() && logits.dim() == 2 && logits.is_contiguous());
  TORCH_CHECK(logits.scalar_type() == torch::kBFloat16 || logits.scalar_type() == torch::kFloat32);
  const int64_t N = logits.size(0), E = logits.size(1);
  c10::cuda::CUDAGuard guard(logits.device());
  auto f32 = logits.options().dtype(torch::kFloat32);
  auto scores = torch::empty({N, E}, f32);
  auto idx = torch::empty({N, top_k}, logits.options().dtype(torch::kInt64));
  auto w = torch::empty({N, top_k}, f32);
  const bool bf = logits.scalar_type() == torch::kBFloat16;
  if (kind == 0) {
    TORCH_CHECK(bias && bias->scalar_type() == torch::kFloat32 && bias->numel() == E);
    mt::router_sigmoid_group(logits.data_ptr(), bf, bias->data_ptr<float>(), scores.data_ptr<float>(),
                             idx.data_ptr<int64_t>(), w.data_ptr<float>(), (int)N, (int)E, (int)top_k, (int)n_group,
                             (int)topk_group, norm, (float)scaling, cur_stream());
  } else {
    mt::router_softmax_topk(logits.data_ptr(), bf, scores.data_ptr<float>(), idx.data_ptr<int64_t>(), w.data_ptr<float>(),
                            (int)N, (int)E, (int)top_k, norm, (float)scaling, cur_stream());
  }
  return {idx, w, scores};
}

torch::Tensor moe_router_bwd(const torch::Tensor& scores, const torch::Tensor& idx, const c10::optional<torch::Tensor>& dw,
                             const c10::optional<torch::Tensor>& dscores, int64_t kind, bool norm, double scaling) {
  const int64_t N = scores.size(0), E = scores.size(1), K = idx.size(1);
  TORCH_CHECK(scores.is_contiguous() && idx.is_contiguous());
  TORCH_CHECK(!dw || (dw->is_contiguous() && dw->scalar_type() == torch::kFloat32));
  TORCH_CHECK(!dscores || (dscores->is_contiguous() && dscores->scalar_type() == torch::kFloat32));
  c10::cuda::CUDAGuard guard(scores.device());
  auto dlogits = torch::empty({N, E}, scores.options());
  mt::router_bwd(kind == 1, scores.data_ptr<float>(), idx.data_ptr<int64_t>(), dw ? dw->data_ptr<float>() : nullptr,
                 dscores ? dscores->data_ptr<float>() : nullptr, dlogits.data_ptr<float>(), (int)N, (int)E, (int)K, norm,
                 (float)scaling, cur_stream());
  return dlogits;
}

// -> (sizes int64 [E], off_p int32 [E+1], pos int64 [M], src int32 [cap])
std::vector<torch::Tensor> moe_sort(const torch::Tensor& experts, int64_t E, int64_t cap) {
  TORCH_CHECK(experts.is_cuda() && experts.is_contiguous() && experts.scalar_type() == torch::kInt64 && E <= 4096);
  const int64_t M = experts.numel();
  c10::cuda::CUDAGuard guard(experts.device());
  auto i32 = experts.options().dtype(torch::kInt32);
  auto chunk_counts = torch::empty({std::max<int64_t>(mt::moe_sort_chunks((int)M), 1) * E}, i32);
  auto sizes = torch::empty({E}, experts.options());
  auto off_p = torch::empty({E + 1}, i32);
  auto pos = torch::empty({M}, experts.options());
  auto src = torch::empty({cap}, i32);
  mt::moe_sort(experts.data_ptr<int64_t>(), (int)M, (int)E, cap, chunk_counts.data_ptr<int>(), sizes.data_ptr<int64_t>(),
               off_p.data_ptr<int>(), pos.data_ptr<int64_t>(), src.data_ptr<int>(), cur_stream());
  return {sizes, off_p, pos, src};
}

torch::Tensor moe_gather_rows(const torch::Tensor& x, const torch::Tensor& src, const c10::optional<torch::Tensor>& w,
                              int64_t K) {
  TORCH_CHECK(x.is_contiguous() && x.scalar_type() == torch::kBFloat16 && x.dim() == 2 && x.size(1) % 8 == 0);
  TORCH_CHECK(src.scalar_type() == torch::kInt32 && src.is_contiguous());
  TORCH_CHECK(!w || (w->scalar_type() == torch::kFloat32 && w->is_contiguous()));
  c10::cuda::CUDAGuard guard(x.device());
  auto rows = torch::empty({src.numel(), x.size(1)}, x.options());
  mt::moe_gather_rows(x.data_ptr(), src.data_ptr<int>(), w ? w->data_ptr<float>() : nullptr, rows.data_ptr(), src.numel(),
                      (int)K, (int)x.size(1), x.size(0) * K, cur_stream());
  return rows;
}

// -> (out [N, D] bf16 or undefined, dw [N, K] fp32 or undefined)
void ep_push_counts(const torch::Tensor& counts, const std::vector<int64_t>& table_ptrs, int64_t rank, int64_t parity) {
  TORCH_CHECK(counts.is_cuda() && counts.is_contiguous() && counts.scalar_type() == torch::kInt64);
  TORCH_CHECK(counts.numel() <= mt::ep_count_slots() && (parity == 0 || parity == 1));
  c10::cuda::CUDAGuard guard(counts.device());
  mt::ep_push_counts(counts.data_ptr<int64_t>(), to_peers(table_ptrs), (int)rank, (int)table_ptrs.size(),
                     (int)counts.numel(), (int)parity, cur_stream());
}

// -> (dst_rank int32 [NK], dst_pos int64 [NK], home_pos int64 [NK], off_local int32 [El+1], tags int32 [NK, 4])
std::vector<torch::Tensor> ep_plan(const torch::Tensor& flat, const torch::Tensor& pos_l, const torch::Tensor& off_l,
                                   const torch::Tensor& w, const torch::Tensor& table, int64_t parity, int64_t rank,
                                   int64_t R, int64_t E, int64_t cap, int64_t K, torch::Tensor& dropped) {
  TORCH_CHECK(flat.is_contiguous() && flat.scalar_type() == torch::kInt64 && pos_l.is_contiguous() &&
              pos_l.scalar_type() == torch::kInt64 && pos_l.numel() == flat.numel());
  TORCH_CHECK(off_l.scalar_type() == torch::kInt32 && off_l.is_contiguous() && off_l.numel() >= E);
  TORCH_CHECK(w.scalar_type() == torch::kFloat32 && w.is_contiguous() && w.numel() == flat.numel());
  TORCH_CHECK(table.scalar_type() == torch::kInt32 && table.is_contiguous() &&
              table.numel() >= 2 * mt::kMaxPeers * mt::ep_count_slots());
  TORCH_CHECK(E % R == 0 && E <= mt::ep_count_slots() && R <= mt::kMaxPeers && dropped.scalar_type() == torch::kInt64);
  c10::cuda::CUDAGuard guard(flat.device());
  const int64_t NK = flat.numel(), El = E / R;
  auto i32 = flat.options().dtype(torch::kInt32);
  auto dst_rank = torch::empty({NK}, i32);
  auto dst_pos = torch::empty({NK}, flat.options());
  auto home_pos = torch::empty({NK}, flat.options());
  auto off_local = torch::empty({El + 1}, i32);
  auto tags = torch::empty({NK, 4}, i32);
  mt::ep_plan(flat.data_ptr<int64_t>(), pos_l.data_ptr<int64_t>(), off_l.data_ptr<int>(), w.data_ptr<float>(),
              table.data_ptr<int>() + parity * mt::kMaxPeers * mt::ep_count_slots(), (int)rank, (int)R, (int)E, (int)El, cap,
              (int)K, NK, dst_rank.data_ptr<int>(), dst_pos.data_ptr<int64_t>(), home_pos.data_ptr<int64_t>(),
              off_local.data_ptr<int>(), tags.data_ptr<int>(),
              reinterpret_cast<unsigned long long*>(dropped.data_ptr<int64_t>()), cur_stream());
  return {dst_rank, dst_pos, home_pos, off_local, tags};
}

// tags int32 [cap, 4] -> (row_src int64 [cap], row_dst int64 [cap], scale fp32 [cap])
std::vector<torch::Tensor> ep_resolve(const torch::Tensor& tags, const std::vector<int64_t>& in_ptrs,
                                      const std::vector<int64_t>& out_ptrs, int64_t row_bytes) {
  TORCH_CHECK(tags.is_cuda() && tags.is_contiguous() && tags.scalar_type() == torch::kInt32 && tags.dim() == 2 &&
              tags.size(1) == 4 && in_ptrs.size() == out_ptrs.size());
  c10::cuda::CUDAGuard guard(tags.device());
  const int64_t cap = tags.size(0);
  auto i64 = tags.options().dtype(torch::kInt64);
  auto row_src = torch::empty({cap}, i64), row_dst = torch::empty({cap}, i64);
  auto scale = torch::empty({cap}, tags.options().dtype(torch::kFloat32));
  mt::ep_resolve(tags.data_ptr<int>(), to_peers(in_ptrs), to_peers(out_ptrs), cap, row_bytes,
                 reinterpret_cast<unsigned long long*>(row_src.data_ptr<int64_t>()),
                 reinterpret_cast<unsigned long long*>(row_dst.data_ptr<int64_t>()), scale.data_ptr<float>(), cur_stream());
  return {row_src, row_dst, scale};
}

int64_t ep_count_slots() { return mt::ep_count_slots(); }

std::vector<torch::Tensor> moe_combine_rows(const torch::Tensor& y, const torch::Tensor& pos,
                                            const c10::optional<torch::Tensor>& w, int64_t N, int64_t K, bool want_out,
                                            const c10::optional<torch::Tensor>& g) {
  TORCH_CHECK(y.is_contiguous() && y.scalar_type() == torch::kBFloat16 && y.size(1) % 8 == 0);
  TORCH_CHECK(pos.scalar_type() == torch::kInt64 && pos.is_contiguous() && pos.numel() == N * K);
  TORCH_CHECK(!w || (w->scalar_type() == torch::kFloat32 && w->is_contiguous() && w->numel() == N * K));
  TORCH_CHECK(!g || (g->scalar_type() == torch::kBFloat16 && g->is_contiguous() && g->size(0) == N && g->size(1) == y.size(1)));
  c10::cuda::CUDAGuard guard(y.device());
  torch::Tensor out, dw;
  if (want_out) out = torch::empty({N, y.size(1)}, y.options());
  if (g) dw = torch::empty({N, K}, y.options().dtype(torch::kFloat32));
  mt::moe_combine_rows(y.data_ptr(), pos.data_ptr<int64_t>(), w ? w->data_ptr<float>() : nullptr,
                       want_out ? out.data_ptr() : nullptr, g ? g->data_ptr() : nullptr,
                       g ? dw.data_ptr<float>() : nullptr, (int)N, (int)K, (int)y.size(1), y.size(0), cur_stream());
  return {out, dw};
}

// out[T, N] = gather(shards)[T, K] @ (b_kn ? B[K, N] : B[N, K]^T); fills `gathered` on the way.
void tp_gemm_ag(const std::vector<int64_t>& shard_ptrs, torch::Tensor& gathered, const torch::Tensor& B, torch::Tensor& out,
                bool b_kn, int64_t rank, torch::Tensor& ready, torch::Tensor& status) {
  TORCH_CHECK(gathered.is_contiguous() && B.is_contiguous() && out.is_contiguous());
  TORCH_CHECK(gathered.scalar_type() == torch::kBFloat16 && B.scalar_type() == torch::kBFloat16 &&
              out.scalar_type() == torch::kBFloat16);
  const int64_t T = gathered.size(0), K = gathered.size(1);
  const int64_t N = b_kn ? B.size(1) : B.size(0);
  TORCH_CHECK((b_kn ? B.size(0) : B.size(1)) == K && out.size(0) == T && out.size(1) == N);
  TORCH_CHECK(K % 64 == 0 && N % 8 == 0 && ready.numel() >= T / 128 && ready.scalar_type() == torch::kInt32);
  c10::cuda::CUDAGuard guard(out.device());
  mt::tp_gemm_ag(to_peers(shard_ptrs), gathered.data_ptr(), B.data_ptr(), out.data_ptr(), (int)T, (int)N, (int)K, (int)rank,
                 (int)shard_ptrs.size(), b_kn, ready.data_ptr<int>(), (int)(128 * K * 2 / 8192), status.data_ptr<int>(),
                 sm_count(), cur_stream());
}

// Partial products of all T rows; rows owned by rank i land in slot_ptrs[i] (its staging slot for this rank).
void tp_gemm_rs(const torch::Tensor& A, const torch::Tensor& B, const std::vector<int64_t>& slot_ptrs, bool b_kn,
                int64_t rank, torch::Tensor& status) {
  TORCH_CHECK(A.is_contiguous() && B.is_contiguous() && A.scalar_type() == torch::kBFloat16 &&
              B.scalar_type() == torch::kBFloat16);
  const int64_t T = A.size(0), K = A.size(1);
  const int64_t N = b_kn ? B.size(1) : B.size(0);
  TORCH_CHECK((b_kn ? B.size(0) : B.size(1)) == K && K % 8 == 0 && N % 8 == 0);
  c10::cuda::CUDAGuard guard(A.device());
  mt::tp_gemm_rs(A.data_ptr(), B.data_ptr(), to_peers(slot_ptrs), (int)T, (int)N, (int)K, (int)rank, (int)slot_ptrs.size(),
                 b_kn, status.data_ptr<int>(), sm_count(), cur_stream());
}

// out[T,N] = a[T,K] @ W[K,N], W gathered inside the kernel from the ranks' row shards into w_full
void fsdp_gemm_agw(const torch::Tensor& a, const std::vector<int64_t>& shard_ptrs, torch::Tensor& w_full, torch::Tensor& out,
                   int64_t rank, torch::Tensor& ready, torch::Tensor& status) {
  TORCH_CHECK(a.is_contiguous() && w_full.is_contiguous() && out.is_contiguous());
  TORCH_CHECK(a.scalar_type() == torch::kBFloat16 && w_full.scalar_type() == torch::kBFloat16 &&
              out.scalar_type() == torch::kBFloat16);
  const int64_t T = a.size(0), K = a.size(1), N = w_full.size(1);
  TORCH_CHECK(w_full.size(0) == K && out.size(0) == T && out.size(1) == N && ready.numel() >= K / 64 &&
              ready.scalar_type() == torch::kInt32);
  c10::cuda::CUDAGuard guard(a.device());
  mt::fsdp_gemm_agw(a.data_ptr(), to_peers(shard_ptrs), w_full.data_ptr(), out.data_ptr(), (int)T, (int)N, (int)K, (int)rank,
                    (int)shard_ptrs.size(), ready.data_ptr<int>(), status.data_ptr<int>(), sm_count(), cur_stream());
}

void tp_reduce_slots(const torch::Tensor& staging, torch::Tensor& y) {
  TORCH_CHECK(staging.is_contiguous() && y.is_contiguous() && staging.scalar_type() == torch::kBFloat16 &&
              y.scalar_type() == torch::kBFloat16 && y.numel() % 8 == 0 && staging.numel() % y.numel() == 0);
  c10::cuda::CUDAGuard guard(y.device());
  mt::tp_reduce_slots(staging.data_ptr(), y.data_ptr(), (int)(staging.numel() / y.numel()), y.numel(), cur_stream());
}

}  // namespace

// ---- debug-bounds registry (common/bounds.cuh): translation units built with -DMINTEXT_DEBUG_BOUNDS register here
namespace mt {
namespace {
struct BoundsUnit { std::string file; BoundsReadFn read; BoundsResetFn reset; };
std::vector<BoundsUnit>& bounds_units() {
  static std::vector<BoundsUnit> units;
  return units;
}
}  // namespace
void register_bounds_unit(const char* file, BoundsReadFn read, BoundsResetFn reset) {
  bounds_units().push_back({std::string(file), read, reset});
}
}  // namespace mt

// [(file, line, index, limit)] for every translation unit that recorded an out-of-range index; empty = clean.
// In the ordinary build no unit registers and the list is always empty.
std::vector<std::tuple<std::string, int64_t, int64_t, int64_t>> debug_bounds_report() {
  std::vector<std::tuple<std::string, int64_t, int64_t, int64_t>> out;
  for (auto& u : mt::bounds_units()) {
    mt::BoundsRecord r{0, 0, 0, 0};
    if (u.read(&r) != 0) throw std::runtime_error("debug_bounds_report: could not read the record of " + u.file);
    if (r.code != 0) out.emplace_back(u.file, (int64_t)r.line, (int64_t)r.index, (int64_t)r.limit);
  }
  return out;
}
void debug_bounds_reset() {
  for (auto& u : mt::bounds_units()) u.reset();
}
int64_t debug_bounds_units() { return (int64_t)mt::bounds_units().size(); }

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("gemm", &gemm, "bf16 tcgen05 GEMM");
  m.def("rmsnorm_fwd", &rmsnorm_fwd);
  m.def("rmsnorm_bwd", &rmsnorm_bwd);
  m.def("rope", &rope);
  m.def("rope_apply", &rope_apply);
  m.def("gated_act_fwd", &gated_act_fwd);
  m.def("gated_act_bwd", &gated_act_bwd);
  m.def("gate_mul_fwd", &gate_mul_fwd);
  m.def("gate_mul_bwd", &gate_mul_bwd);
  m.def("cross_entropy", &cross_entropy);
  m.def("debug_bounds_report", &debug_bounds_report);
  m.def("debug_bounds_reset", &debug_bounds_reset);
  m.def("debug_bounds_units", &debug_bounds_units);
  m.def("threefry_randint", &threefry_randint);
  m.def("embedding_fwd", &embedding_fwd);
  m.def("embedding_bwd", &embedding_bwd);
  m.def("adamw_step", &adamw_step);
  m.def("sumsq", &sumsq);
  m.def("symm_barrier", &symm_barrier);
  m.def("grad_pull_reduce", &grad_pull_reduce);
  m.def("grad_pull_bucket", &grad_pull_bucket);
  m.def("bucket_flag_slots", &bucket_flag_slots);
  m.def("bucket_ready", &bucket_ready);
  m.def("peer_gather", &peer_gather);
  m.def("adamw_publish", &adamw_publish);
  m.def("set_grouped_variant", [](int64_t v) { mt::set_grouped_variant((int)v); });
  m.def("grouped_gemm", &grouped_gemm);
  m.def("grouped_wgrad", &grouped_wgrad);
  m.def("grouped_gemm_scatter", &grouped_gemm_scatter);
  m.def("ep_push_rows", &ep_push_rows);
  m.def("ep_pull_rows", &ep_pull_rows);
  m.def("ep_gather_rows", &ep_gather_rows);
  m.def("gemm_pair", &gemm_pair);
  m.def("gemm_gate_up_act", &gemm_gate_up_act);
  m.def("gemm_gated_bwd", &gemm_gated_bwd);
  m.def("fp8_quantize", &fp8_quantize);
  m.def("gemm_fp8", &gemm_fp8);
  m.def("mxfp8_quantize", &mxfp8_quantize);
  m.def("gemm_mxfp8", &gemm_mxfp8);
  m.def("mxfp8_quantize_stack", &mxfp8_quantize_stack);
  m.def("grouped_gemm_mxfp8", &grouped_gemm_mxfp8);
  m.def("gdn_scan_fwd", &gdn_scan_fwd);
  m.def("gdn_scan_bwd", &gdn_scan_bwd);
  m.def("gdn_prep_fwd", &gdn_prep_fwd);
  m.def("gdn_prep_bwd", &gdn_prep_bwd);
  m.def("conv1d_silu_fwd", &conv1d_silu_fwd);
  m.def("conv1d_silu_bwd", &conv1d_silu_bwd);
  m.def("moe_router", &moe_router);
  m.def("moe_router_bwd", &moe_router_bwd);
  m.def("moe_sort", &moe_sort);
  m.def("moe_gather_rows", &moe_gather_rows);
  m.def("moe_combine_rows", &moe_combine_rows);
  m.def("ep_push_counts", &ep_push_counts);
  m.def("ep_plan", &ep_plan);
  m.def("ep_resolve", &ep_resolve);
  m.def("ep_count_slots", &ep_count_slots);
  m.def("tp_gemm_ag", &tp_gemm_ag);
  m.def("tp_gemm_rs", &tp_gemm_rs);
  m.def("tp_reduce_slots", &tp_reduce_slots);
  m.def("fsdp_gemm_agw", &fsdp_gemm_agw);
  m.def("flash_fwd", &flash_fwd);
  m.def("flash_bwd", &flash_bwd);
}
