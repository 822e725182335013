"""Randomised small-shape differential tests (hypothesis): kernel front-ends against the fp32 oracle on shapes the
fixed-shape tests do not enumerate - ragged tile edges, single rows, narrow and wide feature dims."""

import pytest
import torch
from hypothesis import given, settings
from hypothesis import strategies as st

pytestmark = pytest.mark.gpu
SETTINGS = dict(max_examples=20, deadline=None, derandomize=True)


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-6)).item()


@settings(**SETTINGS)
@given(m=st.integers(1, 700), n8=st.integers(1, 80), k8=st.integers(1, 80), seed=st.integers(0, 1000))
def test_linear_random_shapes(m, n8, k8, seed):
    from mintext_b200.ops import functional as F
    from mintext_b200.ops._ext import check_status

    n, k = 8 * n8, 8 * k8
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(m, k, device="cuda", generator=g).bfloat16().requires_grad_(True)
    w = (torch.randn(k, n, device="cuda", generator=g) * k ** -0.5).bfloat16().requires_grad_(True)
    y = F.linear(x, w)
    dy = torch.randn(m, n, device="cuda", generator=g).bfloat16()
    y.backward(dy)
    torch.cuda.synchronize()
    check_status()
    xf, wf = x.detach().float(), w.detach().float()
    assert _rel(y, xf @ wf) < 1e-2
    assert _rel(x.grad, dy.float() @ wf.t()) < 1e-2
    assert _rel(w.grad, xf.t() @ dy.float()) < 1e-2


@settings(**SETTINGS)
@given(rows=st.integers(1, 300), d8=st.integers(1, 512), seed=st.integers(0, 1000))
def test_rmsnorm_random_shapes(rows, d8, seed):
    from mintext_b200.ops import functional as F
    from mintext_b200.ops import oracle
    from mintext_b200.ops._ext import check_status

    d = 8 * d8
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(rows, d, device="cuda", generator=g).bfloat16().requires_grad_(True)
    scale = (1 + 0.1 * torch.randn(d, device="cuda", generator=g)).requires_grad_(True)
    y = F.rms_norm(x, scale, 1e-5)
    dy = torch.randn(rows, d, device="cuda", generator=g).bfloat16()
    y.backward(dy)
    torch.cuda.synchronize()
    check_status()
    xr, sr = x.detach().float().requires_grad_(True), scale.detach().clone().requires_grad_(True)
    with F.backend("oracle"):
        ref = oracle.rms_norm(xr, sr, 1e-5)
    ref.backward(dy.float())
    assert _rel(y, ref) < 1e-2
    assert _rel(x.grad, xr.grad) < 2e-2
    assert _rel(scale.grad, sr.grad) < 2e-2


@settings(**SETTINGS)
@given(rows=st.integers(1, 500), i8=st.integers(1, 300), act=st.sampled_from(["silu", "gelu_pytorch_tanh", "gelu", "relu"]),
       seed=st.integers(0, 1000))
def test_gated_act_random_shapes(rows, i8, act, seed):
    from mintext_b200.ops import functional as F
    from mintext_b200.ops import oracle
    from mintext_b200.ops._ext import check_status

    inter = 8 * i8
    g = torch.Generator(device="cuda").manual_seed(seed)
    gu = torch.randn(rows, 2 * inter, device="cuda", generator=g).bfloat16().requires_grad_(True)
    y = F.gated_act(gu, act)
    dy = torch.randn(rows, inter, device="cuda", generator=g).bfloat16()
    y.backward(dy)
    torch.cuda.synchronize()
    check_status()
    gr = gu.detach().float().requires_grad_(True)
    ref = oracle.gated_act(gr, act)
    ref.backward(dy.float())
    assert _rel(y, ref) < 1e-2
    assert _rel(gu.grad, gr.grad) < 2e-2


@settings(**SETTINGS)
@given(b=st.integers(1, 2), s128=st.integers(1, 5), hkv=st.integers(1, 3), group=st.integers(1, 3),
       shape=st.sampled_from([(64, 64), (128, 128), (256, 256), (192, 128)]), causal=st.booleans(),
       window=st.sampled_from([None, 96, 200]), softcap=st.sampled_from([None, 30.0]), seed=st.integers(0, 1000))
def test_attention_random_shapes(b, s128, hkv, group, shape, causal, window, softcap, seed):
    from mintext_b200.ops import oracle
    from mintext_b200.ops._ext import check_status
    from mintext_b200.ops.attention import flash_attention

    d, dv = shape
    S, H = 128 * s128, hkv * group
    if window is not None and not causal:
        window = None
    g = torch.Generator(device="cuda").manual_seed(seed)
    q = torch.randn(b, S, H, d, device="cuda", generator=g).bfloat16().requires_grad_(True)
    k = torch.randn(b, S, hkv, d, device="cuda", generator=g).bfloat16().requires_grad_(True)
    v = torch.randn(b, S, hkv, dv, device="cuda", generator=g).bfloat16().requires_grad_(True)
    scale = d ** -0.5
    o = flash_attention(q, k, v, scale, causal, window, softcap)
    do = torch.randn(o.shape, device="cuda", generator=g).bfloat16()
    o.backward(do)
    torch.cuda.synchronize()
    check_status()
    qf, kf, vf = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    ref = oracle.attention(qf, kf, vf, scale, causal, window, softcap)
    ref.backward(do.float())
    assert _rel(o, ref) < 2e-2
    assert _rel(v.grad, vf.grad) < 3e-2
    assert _rel(k.grad, kf.grad) < 3e-2
    assert _rel(q.grad, qf.grad) < 3e-2


@settings(**SETTINGS)
@given(sizes=st.lists(st.integers(0, 300), min_size=1, max_size=9), k8=st.integers(1, 40), n8=st.integers(1, 60),
       seed=st.integers(0, 1000))
def test_grouped_matmul_random_groups(sizes, k8, n8, seed):
    from mintext_b200.ops import moe as moe_ops
    from mintext_b200.ops._ext import check_status

    if sum(sizes) == 0:
        sizes = sizes[:-1] + [5]
    K, N, E = 8 * k8, 8 * n8, len(sizes)
    g = torch.Generator(device="cuda").manual_seed(seed)
    M = sum(sizes)
    x = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    w = (torch.randn(E, K, N, device="cuda", generator=g) * K ** -0.5).bfloat16()
    gs = torch.tensor(sizes, device="cuda")
    y = moe_ops.grouped_matmul_cuda(x, w, gs)
    dw = moe_ops.tgmm_cuda(x, y, gs)
    torch.cuda.synchronize()
    check_status()
    ref = torch.zeros(M, N, device="cuda")
    dw_ref = torch.zeros(E, K, N, device="cuda")
    r0 = 0
    for e, n in enumerate(sizes):
        ref[r0:r0 + n] = x[r0:r0 + n].float() @ w[e].float()
        dw_ref[e] = x[r0:r0 + n].float().t() @ y[r0:r0 + n].float()
        r0 += n
    assert _rel(y, ref) < 1e-2
    assert _rel(dw, dw_ref) < 2e-2


@settings(**SETTINGS)
@given(n=st.integers(1, 600), d8=st.integers(1, 40), v=st.integers(9, 3000), is_vd=st.booleans(),
       ls=st.sampled_from([0.0, 0.1]), zw=st.sampled_from([0.0, 1e-3]), cap=st.sampled_from([None, 30.0]),
       seed=st.integers(0, 1000))
def test_linear_cross_entropy_random_shapes(n, d8, v, is_vd, ls, zw, cap, seed):
    from mintext_b200.ops import functional as F
    from mintext_b200.ops import oracle
    from mintext_b200.ops._ext import check_status

    d = 8 * d8
    g = torch.Generator(device="cuda").manual_seed(seed)
    h = torch.randn(n, d, device="cuda", generator=g).bfloat16().requires_grad_(True)
    w = (torch.randn((v, d) if is_vd else (d, v), device="cuda", generator=g) * d ** -0.5).bfloat16().requires_grad_(True)
    if not is_vd and v % 8 != 0:
        return  # [hidden, vocab] storage needs a 16-byte row pitch
    t = torch.randint(0, v, (n,), device="cuda", generator=g)
    scale = 1.0 / n
    per_tok, z = F.linear_cross_entropy(h, w, t, weight_is_vd=is_vd, label_smoothing=ls, z_loss_weight=zw, softcap=cap,
                                        chunk_rows=256, loss_scale=scale)
    (per_tok.sum() * scale).backward()
    torch.cuda.synchronize()
    check_status()
    hf, wf = h.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    logits = hf @ (wf.t() if is_vd else wf)
    if cap is not None:
        logits = torch.tanh(logits / cap) * cap
    ref, _ = oracle.cross_entropy(logits, t, ls, zw)
    (ref.sum() * scale).backward()
    assert _rel(per_tok, ref) < 2e-2
    assert _rel(h.grad, hf.grad) < 4e-2
    assert _rel(w.grad, wf.grad) < 4e-2


@settings(**SETTINGS)
@given(n=st.integers(16, 400), e=st.integers(2, 12), topk=st.integers(1, 2), d8=st.integers(4, 40), i8=st.integers(2, 30),
       seed=st.integers(0, 1000))
def test_routed_experts_random_shapes(n, e, topk, d8, i8, seed):
    """Counting-sort dispatch, grouped GEMMs, gated activation and weighted combine against the dense per-token sum."""
    from mintext_b200.ops import moe as moe_ops
    from mintext_b200.ops._ext import check_status

    D, I = 8 * d8, 8 * i8
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(n, D, device="cuda", generator=g).bfloat16().requires_grad_(True)
    gu = (torch.randn(e, D, 2 * I, device="cuda", generator=g) * D ** -0.5).bfloat16().requires_grad_(True)
    dn = (torch.randn(e, I, D, device="cuda", generator=g) * I ** -0.5).bfloat16().requires_grad_(True)
    scores = torch.rand(n, e, device="cuda", generator=g)
    w, idx = torch.topk(scores, topk, dim=-1)
    w = w.bfloat16().requires_grad_(True)
    y = moe_ops.experts_forward(x, idx, w, gu, dn, "silu")
    dy = torch.randn(n, D, device="cuda", generator=g).bfloat16()
    y.backward(dy)
    torch.cuda.synchronize()
    check_status()
    xf, guf, dnf, wf = (t.detach().float().requires_grad_(True) for t in (x, gu, dn, w))
    ref = torch.zeros(n, D, device="cuda")
    for k in range(topk):
        h = torch.einsum("nd,ndi->ni", xf, guf[idx[:, k]])
        h = torch.nn.functional.silu(h[:, :I]) * h[:, I:]
        ref = ref + wf[:, k:k + 1] * torch.einsum("ni,nid->nd", h, dnf[idx[:, k]])
    ref.backward(dy.float())
    assert _rel(y, ref) < 2e-2
    assert _rel(x.grad, xf.grad) < 3e-2
    assert _rel(w.grad, wf.grad) < 6e-2   # each entry is one dot product of bf16-rounded rows: cancellation
    assert _rel(gu.grad, guf.grad) < 3e-2
    assert _rel(dn.grad, dnf.grad) < 3e-2


@settings(**SETTINGS)
@given(m=st.integers(1, 700), n8=st.integers(1, 120), k128=st.integers(1, 6), seed=st.integers(0, 1000))
def test_mxfp8_gemm_random_shapes(m, n8, k128, seed):
    """Block-scaled GEMM on ragged M / N (partial 128-row and 192-column tiles) against the product of the
    de-quantised operands."""
    from tests.test_gpu_kernels import _mx_dequant

    from mintext_b200.ops._ext import check_status, ext, status_word

    n, k = 8 * n8, 128 * k128
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = (torch.randn(m, k, device="cuda", generator=g) * torch.logspace(-2, 1, k, device="cuda")).bfloat16()
    w = (torch.randn(n, k, device="cuda", generator=g) * 0.05).bfloat16()
    e = ext()
    xq, xs, _, _ = e.mxfp8_quantize(x, True, False, False, False)
    wq, ws, _, _ = e.mxfp8_quantize(w, True, True, False, False)
    y = e.gemm_mxfp8(xq, xs, wq, ws, status_word(x.device))
    torch.cuda.synchronize()
    check_status()
    ref = _mx_dequant(xq, xs, 128) @ _mx_dequant(wq, ws, 192).t()
    assert _rel(y, ref) < 1e-2


@settings(**SETTINGS)
@given(b=st.integers(1, 3), s=st.integers(1, 300), h=st.integers(1, 6), d=st.sampled_from([32, 64, 128, 192, 256]),
       frac=st.sampled_from([1.0, 0.5, 0.25]), default=st.booleans(), seed=st.integers(0, 1000))
def test_rope_random_shapes(b, s, h, d, frac, default, seed):
    from mintext_b200.ops import functional as F
    from mintext_b200.ops import oracle
    from mintext_b200.ops._ext import check_status

    rot = int(d * frac) // 2 * 2
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(b, s, h, d, device="cuda", generator=g).bfloat16().requires_grad_(True)
    inv_freq = 1.0 / (10000.0 ** (torch.arange(0, rot, 2, device="cuda").float() / rot))
    tables = oracle.rope_tables(inv_freq, 1.0, 512, device="cuda")
    if default:
        pos = torch.arange(s, device="cuda")[None].expand(b, -1)
    else:
        pos = torch.randint(0, 512, (b, s), device="cuda", generator=g)
    y = F.rope(x, pos, inv_freq, 1.0, rot, False, tables=tables, default_positions=default)
    dy = torch.randn(y.shape, device="cuda", generator=g).bfloat16()
    y.backward(dy)
    torch.cuda.synchronize()
    check_status()
    xf = x.detach().float().requires_grad_(True)
    ref = oracle.apply_rope(xf, pos, inv_freq, 1.0, rot, False)
    ref.backward(dy.float())
    assert _rel(y, ref) < 1e-2
    assert _rel(x.grad, xf.grad) < 1e-2


@settings(**SETTINGS)
@given(b=st.integers(1, 3), s=st.integers(1, 200), c8=st.integers(1, 64), k=st.integers(2, 4), seed=st.integers(0, 1000))
def test_conv1d_silu_random_shapes(b, s, c8, k, seed):
    from mintext_b200.ops import functional as F
    from mintext_b200.ops import oracle
    from mintext_b200.ops._ext import check_status

    c = 8 * c8
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(b, s, c, device="cuda", generator=g).bfloat16().requires_grad_(True)
    w = (torch.randn(c, 1, k, device="cuda", generator=g) * 0.5).bfloat16().requires_grad_(True)
    y = F.causal_conv1d_silu(x, w)
    dy = torch.randn(y.shape, device="cuda", generator=g).bfloat16()
    y.backward(dy)
    torch.cuda.synchronize()
    check_status()
    xr, wr = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    ref = torch.nn.functional.silu(oracle.causal_conv1d(xr, wr))
    ref.backward(dy.float())
    assert _rel(y, ref) < 1e-2
    assert _rel(x.grad, xr.grad) < 2e-2
    assert _rel(w.grad, wr.grad) < 3e-2


@settings(**SETTINGS)
@given(n=st.integers(1, 500), v=st.integers(2, 4000), d8=st.integers(1, 64), scale=st.sampled_from([None, 8.0]),
       seed=st.integers(0, 1000))
def test_embedding_random_shapes(n, v, d8, scale, seed):
    from mintext_b200.ops import functional as F
    from mintext_b200.ops._ext import check_status

    d = 8 * d8
    g = torch.Generator(device="cuda").manual_seed(seed)
    table = torch.randn(v, d, device="cuda", generator=g).bfloat16().requires_grad_(True)
    ids = torch.randint(0, v, (2, n), device="cuda", generator=g)
    y = F.embedding(table, ids, torch.bfloat16, scale)
    dy = torch.randn(y.shape, device="cuda", generator=g).bfloat16()
    y.backward(dy)
    torch.cuda.synchronize()
    check_status()
    tf = table.detach().float().requires_grad_(True)
    ref = tf[ids] * (scale if scale is not None else 1.0)
    ref.backward(dy.float())
    assert _rel(y, ref) < 1e-2
    assert _rel(table.grad, tf.grad) < 2e-2


@settings(**SETTINGS)
@given(b=st.integers(1, 2), h=st.integers(1, 3), s=st.integers(1, 260), dk=st.sampled_from([64, 128]),
       dv=st.sampled_from([32, 64, 128]), seed=st.integers(0, 1000))
def test_gated_delta_rule_random_shapes(b, h, s, dk, dv, seed):
    from mintext_b200.ops import gdn, oracle
    from mintext_b200.ops._ext import check_status

    g_ = torch.Generator(device="cuda").manual_seed(seed)
    q, k = (torch.randn(b, h, s, dk, device="cuda", generator=g_).requires_grad_(True) for _ in range(2))
    v = torch.randn(b, h, s, dv, device="cuda", generator=g_).requires_grad_(True)
    beta = torch.rand(b, h, s, device="cuda", generator=g_).requires_grad_(True)
    gl = (-torch.rand(b, h, s, device="cuda", generator=g_) * 0.5).requires_grad_(True)
    assert gdn.cuda_path(q, v, 64)
    o = gdn.chunk_gated_delta_rule_cuda(q, k, v, beta, gl)
    do = torch.randn(o.shape, device="cuda", generator=g_)
    o.backward(do)
    torch.cuda.synchronize()
    check_status()
    ins = [t.detach().clone().requires_grad_(True) for t in (q, k, v, beta, gl)]
    ref = oracle.chunk_gated_delta_rule(*ins)
    ref.backward(do)
    assert _rel(o, ref) < 1e-3
    for name, a, r in zip("qkvbg", (q, k, v, beta, gl), ins):
        assert _rel(a.grad, r.grad) < 5e-3, name


@settings(**SETTINGS)
@given(n=st.integers(1, 700), groups=st.sampled_from([1, 2, 4, 8]), per=st.sampled_from([2, 4, 16, 32]),
       topk=st.integers(1, 8), norm=st.booleans(), softmax=st.booleans(), seed=st.integers(0, 1000))
def test_routers_random_shapes(n, groups, per, topk, norm, softmax, seed):
    """Both router kernels against the oracle: same experts, weights, scores, auxiliary loss and logit gradients."""
    from mintext_b200.ops import moe as moe_ops
    from mintext_b200.ops import oracle
    from mintext_b200.ops._ext import check_status

    E = groups * per
    topk_group = max(groups // 2, 1)
    topk = min(topk, topk_group * per)
    g = torch.Generator(device="cuda").manual_seed(seed)
    logits = (torch.randn(n, E, device="cuda", generator=g) * 2).requires_grad_(True)
    bias = torch.randn(E, device="cuda", generator=g) * 0.1
    ref_in = logits.detach().clone().requires_grad_(True)
    if softmax:
        idx, w, probs, aux = moe_ops.router_softmax_topk(logits, topk, norm, 1.5)
        ridx, rw, rprobs, raux = oracle.router_softmax_topk(ref_in, topk, norm, 1.5)
    else:
        idx, w, probs = moe_ops.router_sigmoid_group(logits, bias, topk, groups, topk_group, norm, 2.5)
        ridx, rw, rprobs = oracle.router_sigmoid_group(ref_in, bias, topk, groups, topk_group, norm, 2.5)
        aux = raux = None
    dw = torch.randn(w.shape, device="cuda", generator=g)
    loss = (w.float() * dw).sum() + (aux if aux is not None else 0.0)
    rloss = (rw.float() * dw).sum() + (raux if raux is not None else 0.0)
    loss.backward()
    rloss.backward()
    torch.cuda.synchronize()
    check_status()
    assert torch.equal(idx.long().sort(-1)[0], ridx.long().sort(-1)[0])
    order, rorder = idx.long().argsort(-1), ridx.long().argsort(-1)
    assert torch.allclose(w.float().gather(1, order), rw.float().gather(1, rorder), atol=1e-5, rtol=1e-4)
    assert torch.allclose(probs.float(), rprobs.float(), atol=1e-5)
    if aux is not None:
        assert abs(float(aux) - float(raux)) < 1e-4
    assert _rel(logits.grad, ref_in.grad) < 1e-3
