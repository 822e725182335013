"""tcgen05 grouped GEMMs and the padded MoE pipeline against per-expert loops."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


def _check():
    from mintext_b200.ops._ext import check_status

    torch.cuda.synchronize()
    check_status()


@pytest.mark.parametrize("sizes", [[128, 128, 128, 128], [300, 0, 77, 513], [0, 0, 1000, 1], [5, 6, 7, 8]])
def test_grouped_matmul_and_grads_vs_loop(sizes):
    from mintext_b200 import kernels
    from mintext_b200.ops import oracle

    torch.manual_seed(0)
    E, K, N = len(sizes), 256, 384
    M = sum(sizes)
    gs = torch.tensor(sizes, device="cuda")
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(E, K, N, device="cuda") * 0.05).bfloat16().requires_grad_(True)
    y = kernels.grouped_matmul(x, w, gs)
    ref = oracle.grouped_matmul(x.detach().float(), w.detach().float(), gs)
    _check()
    assert _rel(y, ref) < 1e-2
    dy = torch.randn_like(y)
    y.backward(dy)
    _check()
    dx_ref = oracle.grouped_matmul(dy.float(), w.detach().float().transpose(1, 2), gs)
    dw_ref = oracle.tgmm(x.detach().float(), dy.float(), gs)
    assert _rel(x.grad, dx_ref) < 1e-2
    assert _rel(w.grad, dw_ref) < 1e-2
    t = kernels.tgmm(x.detach(), dy, gs)
    _check()
    assert _rel(t, dw_ref) < 1e-2


def test_moe_block_kernel_path_matches_oracle_path():
    from mintext_b200 import MinTextConfig
    from mintext_b200.modules import MoEBlock
    from mintext_b200.ops import functional as F

    cfg = MinTextConfig(hidden_size=256, num_experts=8, num_experts_per_tok=2, moe_intermediate_size=128, n_group=4,
                        topk_group=2, n_shared_experts=1)
    blk = MoEBlock(cfg, rngs=torch.Generator().manual_seed(0)).cuda()
    for n, p in blk.named_parameters():
        if p.dim() >= 2:
            p.data = p.data.bfloat16()
    x = torch.randn(2, 192, 256, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    out, aux = blk(x)
    params = [p for p in blk.parameters() if p.requires_grad]
    g = torch.autograd.grad(out.float().pow(2).mean(), [x] + params)
    _check()
    with F.backend("oracle"):
        out2, _ = blk(x)
        g2 = torch.autograd.grad(out2.float().pow(2).mean(), [x] + params)
    assert _rel(out, out2) < 2e-2
    for a, b in zip(g, g2):
        assert _rel(a, b) < 5e-2


def test_moe_model_trains_with_engine():
    from mintext_b200 import MinTextConfig
    from mintext_b200.models import Transformer
    from mintext_b200.parallel.engine import TrainEngine

    cfg = MinTextConfig(num_hidden_layers=2, hidden_size=256, num_attention_heads=4, num_key_value_heads=2, head_dim=64,
                        intermediate_size=512, vocab_size=1024, seq_length=128, steps=20, learning_rate=2e-3,
                        num_experts=8, num_experts_per_tok=2, moe_intermediate_size=128, n_group=1, topk_group=1,
                        first_k_dense_replace=1, n_shared_experts=0, router_type="softmax_topk",
                        router_aux_loss_coef=0.01, enable_tensorboard=False, enable_checkpointing=False)
    eng = TrainEngine(Transformer(cfg, rngs=0), cfg, device="cuda")
    tok = torch.randint(0, 1024, (4, 128), device="cuda")
    losses = []
    for _ in range(8):
        out = eng.train_step({"input_tokens": tok, "target_tokens": tok}, num_micro=1)
        losses.append(float(out["loss"]))
    eng.check()
    assert out["moe_expert_counts"].shape == (1, 8)
    assert losses[-1] < losses[1] - 0.3, losses


@pytest.mark.parametrize("E,K,n_group,topk_group,norm", [(64, 6, 8, 3, True), (256, 8, 8, 4, True), (8, 2, 1, 1, False),
                                                         (128, 8, 4, 2, False)])
def test_router_sigmoid_group_kernel_matches_oracle(E, K, n_group, topk_group, norm):
    from mintext_b200.ops import moe as moe_ops
    from mintext_b200.ops import oracle

    torch.manual_seed(1)
    N = 777
    logits = (torch.randn(N, E, device="cuda") * 2).requires_grad_(True)
    bias = torch.randn(E, device="cuda") * 0.1
    idx, w, scores = moe_ops.router_sigmoid_group(logits, bias, K, n_group, topk_group, norm, 2.5)
    lr = logits.detach().clone().requires_grad_(True)
    idx_r, w_r, scores_r = oracle.router_sigmoid_group(lr, bias, K, n_group, topk_group, norm, 2.5)
    _check()
    assert (idx == idx_r).float().mean().item() > 0.999  # fast-math sigmoid may flip a near tie
    same = (idx == idx_r).all(dim=1)
    assert torch.allclose(w[same], w_r[same], atol=1e-5, rtol=1e-4)
    assert torch.allclose(scores, scores_r, atol=1e-6, rtol=1e-5)
    gw, gs = torch.randn_like(w), torch.randn_like(scores) * 0.1
    (w * gw).sum().add((scores * gs).sum()).backward()
    ((w_r * gw).sum() + (scores_r * gs).sum()).backward()
    _check()
    assert torch.allclose(logits.grad[same], lr.grad[same], atol=1e-5, rtol=1e-3)


def test_router_softmax_kernel_matches_oracle():
    from mintext_b200.ops import moe as moe_ops
    from mintext_b200.ops import oracle

    torch.manual_seed(2)
    N, E, K = 500, 128, 8
    logits = torch.randn(N, E, device="cuda").bfloat16().requires_grad_(True)
    idx, w, probs, aux = moe_ops.router_softmax_topk(logits, K, True)
    lr = logits.detach().clone().requires_grad_(True)
    idx_r, w_r, probs_r, aux_r = oracle.router_softmax_topk(lr, K, True)
    _check()
    same = (idx == idx_r).all(dim=1)
    assert same.float().mean().item() > 0.99
    assert torch.allclose(w[same], w_r[same], atol=1e-5, rtol=1e-4)
    assert torch.allclose(probs, probs_r, atol=1e-6, rtol=1e-4)
    assert abs(float(aux) - float(aux_r)) < 1e-4
    gw = torch.randn_like(w)
    ((w * gw).sum() + aux * 3.0).backward()
    ((w_r * gw).sum() + aux_r * 3.0).backward()
    _check()
    assert _rel(logits.grad[same], lr.grad[same]) < 2e-2  # bf16 gradients


@pytest.mark.parametrize("N,K,E", [(1000, 2, 8), (4096, 8, 128), (3, 1, 4), (5000, 4, 640)])
def test_counting_sort_dispatch_matches_stable_argsort(N, K, E):
    from mintext_b200.ops import moe as moe_ops

    torch.manual_seed(3)
    idx = torch.randint(0, E, (N, K), device="cuda")
    if E > 4:
        idx[idx == 1] = 2  # an empty expert
    sizes, off_p, pos, src = moe_ops.sort_by_expert(idx, E)
    _check()
    flat = idx.reshape(-1)
    assert torch.equal(sizes, torch.bincount(flat, minlength=E))
    ref_off_p, ref_off_u = moe_ops.padded_offsets(sizes)
    assert torch.equal(off_p, ref_off_p)
    order = torch.argsort(flat, stable=True)
    dest = moe_ops.row_destinations(flat[order], ref_off_p, ref_off_u)
    ref_pos = torch.empty_like(dest)
    ref_pos[order] = dest
    assert torch.equal(pos, ref_pos)
    live = src >= 0
    assert int(live.sum()) == N * K
    assert torch.equal(pos[src[live].long()], torch.nonzero(live).squeeze(1))


def test_dispatch_combine_kernels_and_grads():
    from mintext_b200.ops import moe as moe_ops

    torch.manual_seed(4)
    N, K, E, D = 512, 4, 16, 256
    idx = torch.stack([torch.randperm(E, device="cuda")[:K] for _ in range(N)])
    x = torch.randn(N, D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = torch.rand(N, K, device="cuda", requires_grad=True)
    sizes, off_p, pos, src = moe_ops.sort_by_expert(idx, E)
    rows = moe_ops._DispatchFn.apply(x, src, pos, K)
    out = moe_ops._CombineFn.apply(rows * 1.0, w, pos, src, K)  # identity experts: out[n] = sum_k w[n,k] x[n]
    _check()
    xr = x.detach().float().requires_grad_(True)
    wr = w.detach().clone().requires_grad_(True)
    ref = xr * wr.sum(1, keepdim=True)
    assert _rel(out, ref) < 1e-2
    assert float(rows[src < 0].abs().max()) == 0.0
    g = torch.randn_like(out)
    out.backward(g)
    ref.backward(g.float())
    _check()
    assert _rel(x.grad, xr.grad) < 2e-2
    assert _rel(w.grad, wr.grad) < 2e-2


def test_grouped_gemm_with_row_scatter_epilogue():
    """The expert GEMM whose epilogue writes every output row to a per-row address (the fused combine of expert
    parallelism), here into a local buffer through a random permutation with some rows dropped."""
    from mintext_b200.ops._ext import check_status, ext, status_word

    torch.manual_seed(0)
    E, K, N = 5, 192, 320
    sizes = torch.tensor([128, 384, 0, 256, 128])
    off = torch.zeros(E + 1, dtype=torch.int32)
    off[1:] = torch.cumsum(sizes, 0)
    M = int(off[-1])
    x = torch.randn(M, K, device="cuda").bfloat16()
    w = (torch.randn(E, K, N, device="cuda") * 0.05).bfloat16()
    off = off.cuda()
    y = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    ext().grouped_gemm(x, w, y, off, True, status_word())
    perm = torch.randperm(M, device="cuda")
    keep = torch.rand(M, device="cuda") > 0.2
    out = torch.full((M, N), 7.0, device="cuda", dtype=torch.bfloat16)
    dst = torch.where(keep, out.data_ptr() + perm * (N * 2), torch.zeros_like(perm)).contiguous()
    ext().grouped_gemm_scatter(x, w, dst, off, True, status_word())
    torch.cuda.synchronize()
    check_status()
    want = torch.full_like(out, 7.0)
    want[perm[keep]] = y[keep]
    assert torch.equal(out, want)



def test_grouped_tilings_select_both_kernel_variants_and_agree():
    """`tiling` picks the single-CTA or the CTA-pair grouped kernel; both give the fp32 product, values and gradients."""
    from mintext_b200 import kernels

    torch.manual_seed(0)
    E, M, K, N = 4, 1024, 256, 512
    sizes = torch.tensor([300, 0, 500, 224], device="cuda")
    x = (torch.randn(M, K, device="cuda") * 0.5).bfloat16()
    w = (torch.randn(E, K, N, device="cuda") * 0.05).bfloat16()
    outs = []
    for tiling in ((128, 64, 256), (256, 64, 256), None):
        xa, wa = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
        y = kernels.grouped_matmul(xa, wa, sizes, tiling=tiling)
        y.backward(torch.ones_like(y))
        outs.append((y.float(), xa.grad.float(), wa.grad.float()))
    ref = torch.cat([x[a:b].float() @ w[e].float() for e, (a, b) in
                     enumerate(zip([0, 300, 300, 800], [300, 300, 800, 1024]))])
    for y, dx, dw in outs:
        assert ((y - ref).norm() / ref.norm()).item() < 1e-2
        assert ((dx - outs[0][1]).norm() / outs[0][1].norm()).item() < 1e-2
        assert ((dw - outs[0][2]).norm() / outs[0][2].norm()).item() < 1e-2


def test_autotuner_times_real_variants_on_gpu(tmp_path):
    from mintext_b200.kernels.autotuner import GPU_TILINGS, MoETuningConfig, autotune_moe

    r = autotune_moe(MoETuningConfig(8, 512, 256, 4096), cache_dir=str(tmp_path), warmup_iters=2, bench_iters=3)
    assert tuple(r.gate_up_tiling) in GPU_TILINGS and tuple(r.down_tiling) in GPU_TILINGS
    assert len(r.throughput_gflops["gate_up_candidates_ms"]) == 2 and r.backend == "tcgen05_grouped"


def _mx_qdq(t):
    """Quantise-dequantise along the last dim in 32-element blocks: e4m3 elements, power-of-two block scale."""
    shape = t.shape
    tf = t.float().reshape(-1, shape[-1] // 32, 32)
    amax = tf.abs().amax(-1, keepdim=True)
    e = torch.ceil(torch.log2(amax.clamp_min(2.0 ** -120) / 448.0)).clamp(-127, 127)
    scale = torch.exp2(e)
    return ((tf / scale).clamp(-448, 448).to(torch.float8_e4m3fn).float() * scale).reshape(shape)


def test_grouped_mxfp8_matches_dequantised_product():
    """Block-scaled expert GEMM: forward and data gradient equal the fp32 product of the de-quantised operands (each
    quantised along the dimension that product contracts); the weight gradient is the bf16 one."""
    from mintext_b200.ops import moe as moe_ops
    from mintext_b200.ops._ext import check_status

    torch.manual_seed(0)
    E, K, N = 4, 256, 384          # N is not a multiple of the 192-row B tile: the ragged tile must not read the next expert
    sizes = [256, 0, 128, 384]
    off = torch.tensor([0, 256, 256, 384, 768], device="cuda", dtype=torch.int32)
    cap = 1024                     # rows beyond the last offset stay unused
    x = (torch.randn(cap, K, device="cuda") * 0.7).bfloat16()
    x[768:] = 0
    w = (torch.randn(E, K, N, device="cuda") * 0.05).bfloat16()
    xa, wa = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
    assert moe_ops.mxfp8_grouped_path(xa, wa)
    y = moe_ops.grouped_padded(xa, wa, off, None, True)
    dy = (torch.randn_like(y.float()) * 0.3).bfloat16()
    dy[768:] = 0
    y.backward(dy)
    torch.cuda.synchronize()
    check_status()
    xq = _mx_qdq(x)                                  # activations: blocks along K
    wq_fwd = _mx_qdq(w.transpose(1, 2)).transpose(1, 2)   # weights for the forward: blocks along K
    wq_bwd = _mx_qdq(w)                              # weights for the data gradient: blocks along N
    dyq = _mx_qdq(dy)
    ref_y = torch.zeros(cap, N, device="cuda")
    ref_dx = torch.zeros(cap, K, device="cuda")
    ref_dw = torch.zeros(E, K, N, device="cuda")
    for e in range(E):
        a, b = int(off[e]), int(off[e + 1])
        ref_y[a:b] = xq[a:b] @ wq_fwd[e]
        ref_dx[a:b] = dyq[a:b] @ wq_bwd[e].t()
        ref_dw[e] = x[a:b].float().t() @ dy[a:b].float()
    rel = lambda g, r: ((g.float() - r).norm() / (r.norm() + 1e-9)).item()
    assert rel(y[:768], ref_y[:768]) < 1e-2, rel(y[:768], ref_y[:768])
    assert rel(xa.grad[:768], ref_dx[:768]) < 1e-2, rel(xa.grad[:768], ref_dx[:768])
    assert rel(wa.grad, ref_dw) < 1e-2, rel(wa.grad, ref_dw)
    # and close to the unquantised bf16 path (quantisation noise only)
    yb = moe_ops.grouped_padded(x, w, off, None, False)
    assert rel(y[:768], yb[:768].float()) < 6e-2


def test_experts_forward_with_fp8_tracks_the_bf16_path():
    from mintext_b200.ops import moe as moe_ops

    torch.manual_seed(1)
    n_tok, E, K, D, I = 512, 8, 2, 256, 128
    x = torch.randn(n_tok, D, device="cuda", dtype=torch.bfloat16)
    idx = torch.randint(0, E, (n_tok, K), device="cuda")
    wts = torch.rand(n_tok, K, device="cuda")
    gu = (torch.randn(E, D, 2 * I, device="cuda") * 0.05).bfloat16()
    dn = (torch.randn(E, I, D, device="cuda") * 0.05).bfloat16()
    a = moe_ops.experts_forward(x, idx, wts, gu, dn, "silu", fp8=False).float()
    b = moe_ops.experts_forward(x, idx, wts, gu, dn, "silu", fp8=True).float()
    assert ((a - b).norm() / a.norm()).item() < 8e-2
