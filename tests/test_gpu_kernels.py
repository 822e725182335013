"""Numerics of the hand-written CUDA kernels against plain PyTorch fp32 references."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ext():
    from mintext_b200.ops._ext import ext

    return ext()


def _status():
    from mintext_b200.ops._ext import status_word

    return status_word()


def _check():
    from mintext_b200.ops._ext import check_status

    torch.cuda.synchronize()
    check_status()


def _rel_err(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


def _tiles(t, tile):
    """[M, N] -> [ceil(M/tile), ceil(N/tile), tile*tile] with zero padding at ragged edges."""
    M, N = t.shape
    Mp, Np = -(-M // tile) * tile, -(-N // tile) * tile
    p = torch.zeros(Mp, Np, device=t.device, dtype=torch.float32)
    p[:M, :N] = t.float()
    return p.view(Mp // tile, tile, Np // tile, tile).permute(0, 2, 1, 3).reshape(Mp // tile, Np // tile, -1)


def _assert_tiles_close(got, ref, tile=128, rel=1e-2, max_abs=2.0 ** -6):
    """Every ``tile x tile`` block of the output on its own: relative Frobenius error below ``rel`` and largest
    absolute error below ``max_abs`` times the block's largest reference magnitude.  A whole-tensor norm hides one
    misplaced epilogue box (a 32 x 64 box is 0.01 % of a 4096 x 2048 output); a per-block bound does not."""
    d, r = _tiles(got.float() - ref.float(), tile), _tiles(ref, tile)
    fro = d.norm(dim=-1) / (r.norm(dim=-1) + 1e-6)
    worst = d.abs().amax(-1) / (r.abs().amax(-1) + 1e-6)
    i = int(fro.argmax())
    assert fro.max().item() < rel, ("tile frobenius", divmod(i, fro.shape[1]), fro.max().item())
    j = int(worst.argmax())
    assert worst.max().item() < max_abs, ("tile max-abs", divmod(j, worst.shape[1]), worst.max().item())


@pytest.mark.parametrize("a_km,b_kn", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (256, 256, 128), (384, 512, 320), (200, 136, 72), (1024, 2048, 1024)])
def test_gemm_layouts(a_km, b_kn, M, N, K):
    torch.manual_seed(0)
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(K, N, device="cuda", dtype=torch.bfloat16)
    ref = a.float() @ b.float()
    A = a.t().contiguous() if a_km else a
    B = b if b_kn else b.t().contiguous()
    c = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    _ext().gemm(A, B, c, a_km, b_kn, False, _status())
    _check()
    assert _rel_err(c, ref) < 1e-2
    _assert_tiles_close(c, ref)


@pytest.mark.parametrize("accumulate", [False, True])
def test_gemm_fp32_out_and_accumulate(accumulate):
    torch.manual_seed(1)
    M, N, K = 512, 384, 256
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    c0 = torch.randn(M, N, device="cuda", dtype=torch.float32)
    c = c0.clone()
    _ext().gemm(a, b, c, False, False, accumulate, _status())
    _check()
    ref = a.float() @ b.float().t() + (c0 if accumulate else 0)
    assert _rel_err(c, ref) < 1e-5
    _assert_tiles_close(c, ref, rel=1e-5, max_abs=1e-5)


@pytest.mark.parametrize("M,N,K,b_kn", [(256, 256, 64, False), (512, 768, 320, True), (384, 520, 1024, False),
                                         (4096, 2048, 2048, True)])
def test_gemm_on_cta_pairs(M, N, K, b_kn):
    """cta_group::2 kernel (256x256 tiles on two SMs) against the fp32 product, ragged edges included."""
    torch.manual_seed(4)
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    ref = a.float() @ b.float().t()
    B = b.t().contiguous() if b_kn else b
    c = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    _ext().gemm_pair(a, B, c, b_kn, _status())
    _check()
    assert _rel_err(c, ref) < 1e-2
    _assert_tiles_close(c, ref)


def test_gemm_weight_gradient_layout_with_split_k():
    """x^T dy accumulated into fp32 with few output tiles and a long contraction: the launcher splits K."""
    torch.manual_seed(3)
    T, Kin, Nout = 4096 + 64, 2048, 3072   # 16 x 12 tiles on 148 SMs -> three K slices (of unequal length)
    x = torch.randn(T, Kin, device="cuda", dtype=torch.bfloat16)
    dy = torch.randn(T, Nout, device="cuda", dtype=torch.bfloat16)
    c0 = torch.randn(Kin, Nout, device="cuda", dtype=torch.float32)
    c = c0.clone()
    _ext().gemm(x, dy, c, True, True, True, _status())
    _check()
    ref = x.float().t() @ dy.float() + c0
    assert _rel_err(c, ref) < 1e-4


def test_gemm_bf16_accumulate():
    torch.manual_seed(2)
    M, N, K = 256, 256, 512
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    c0 = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
    c = c0.clone()
    _ext().gemm(a, b, c, False, False, True, _status())
    _check()
    ref = a.float() @ b.float().t() + c0.float()
    assert _rel_err(c, ref) < 2e-2


def test_gemm_strided_views():
    """Operands and output may be column blocks of wider buffers."""
    torch.manual_seed(3)
    M, N, K = 256, 192, 128
    big_a = torch.randn(M, 3 * K, device="cuda", dtype=torch.bfloat16)
    a = big_a[:, K:2 * K]
    b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    big_c = torch.zeros(M, 2 * N + 64, device="cuda", dtype=torch.bfloat16)
    c = big_c[:, 64:64 + N]
    _ext().gemm(a, b, c, False, False, False, _status())
    _check()
    ref = a.float() @ b.float().t()
    assert _rel_err(c, ref) < 1e-2
    assert big_c[:, :64].abs().max().item() == 0
    assert big_c[:, 64 + N:].abs().max().item() == 0


def test_gemm_large_persistent():
    torch.manual_seed(4)
    M, N, K = 4096, 4096, 2048
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    c = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    _ext().gemm(a, b, c, False, False, False, _status())
    _check()
    ref = (a @ b.t()).float()
    assert _rel_err(c, ref) < 5e-3


def test_rmsnorm_fwd_bwd():
    torch.manual_seed(0)
    rows, dim = 1000, 2048
    x = torch.randn(rows, dim, device="cuda", dtype=torch.bfloat16)
    res = torch.randn(rows, dim, device="cuda", dtype=torch.bfloat16)
    w = (1 + 0.1 * torch.randn(dim, device="cuda")).float()
    y = torch.empty_like(x)
    res_out = torch.empty_like(x)
    rstd = torch.empty(rows, device="cuda")
    e = _ext()
    e.rmsnorm_fwd(x, res, w, y, res_out, rstd, 1e-5)
    h = (x.float() + res.float()).bfloat16()
    assert torch.equal(res_out, h)
    hf = h.float()
    ref_rstd = torch.rsqrt(hf.pow(2).mean(-1) + 1e-5)
    ref = ((hf * ref_rstd[:, None]).bfloat16() * w.bfloat16())
    assert _rel_err(y, ref) < 1e-2
    assert torch.allclose(rstd, ref_rstd, rtol=1e-4)
    # backward vs autograd in fp32
    dy = torch.randn(rows, dim, device="cuda", dtype=torch.bfloat16)
    hx = hf.clone().requires_grad_(True)
    wf = w.clone().requires_grad_(True)
    yy = hx * torch.rsqrt(hx.pow(2).mean(-1, keepdim=True) + 1e-5) * wf
    yy.backward(dy.float())
    dx = torch.empty_like(x)
    parts = torch.empty(64, dim, device="cuda")
    dw = torch.zeros(dim, device="cuda")
    e.rmsnorm_bwd(h, w, rstd, dy, None, dx, parts, dw, False)
    torch.cuda.synchronize()
    assert _rel_err(dx, hx.grad) < 1e-2
    assert _rel_err(dw, wf.grad) < 1e-2


@pytest.mark.parametrize("interleave", [False, True])
def test_rope_roundtrip_and_reference(interleave):
    torch.manual_seed(0)
    B, S, H, dh, rot = 2, 64, 4, 64, 64
    x = torch.randn(B * S, H * dh + 32, device="cuda", dtype=torch.bfloat16)
    x0 = x.clone()
    inv = 1.0 / (10000 ** (torch.arange(0, rot, 2, device="cuda").float() / rot))
    ang = torch.arange(S, device="cuda").float()[:, None] * inv[None]
    cos_t, sin_t = ang.cos().contiguous(), ang.sin().contiguous()
    e = _ext()
    e.rope(x, cos_t, sin_t, None, S, H, dh, rot, interleave, False)
    xr = x0[:, :H * dh].float().view(B, S, H, dh)
    cos = torch.cat([cos_t, cos_t], -1)[None, :, None, :]
    sin = torch.cat([sin_t, sin_t], -1)[None, :, None, :]
    if interleave:
        p = xr.view(B, S, H, dh // 2, 2)
        rotx = torch.stack([-p[..., 1], p[..., 0]], -1).reshape(B, S, H, dh)
    else:
        rotx = torch.cat([-xr[..., dh // 2:], xr[..., :dh // 2]], -1)
    ref = xr * cos + rotx * sin
    assert _rel_err(x[:, :H * dh].view(B, S, H, dh), ref) < 1e-2
    assert torch.equal(x[:, H * dh:], x0[:, H * dh:])
    if not interleave:
        e.rope(x, cos_t, sin_t, None, S, H, dh, rot, interleave, True)
        assert _rel_err(x[:, :H * dh], x0[:, :H * dh]) < 2e-2


@pytest.mark.parametrize("act,fn", [(0, torch.nn.functional.silu), (1, lambda t: torch.nn.functional.gelu(t, approximate="tanh"))])
def test_gated_act(act, fn):
    torch.manual_seed(0)
    rows, inter = 300, 512
    gu = torch.randn(rows, 2 * inter, device="cuda", dtype=torch.bfloat16)
    out = torch.empty(rows, inter, device="cuda", dtype=torch.bfloat16)
    e = _ext()
    e.gated_act_fwd(gu, out, act)
    g = gu.float().requires_grad_(True)
    ref = fn(g[:, :inter]) * g[:, inter:]
    assert _rel_err(out, ref) < 1e-2
    dout = torch.randn_like(out)
    ref.backward(dout.float())
    dgu = torch.empty_like(gu)
    e.gated_act_bwd(gu, dout, dgu, act)
    assert _rel_err(dgu, g.grad) < 1e-2


@pytest.mark.parametrize("ls,zw", [(0.0, 0.0), (0.1, 1e-3)])
def test_cross_entropy(ls, zw):
    torch.manual_seed(0)
    rows, V = 64, 4104
    logits = (3 * torch.randn(rows, V, device="cuda")).bfloat16()
    tgt = torch.randint(0, V, (rows,), device="cuda")
    lf = logits.float().requires_grad_(True)
    lse = torch.logsumexp(lf, -1)
    logp = lf - lse[:, None]
    nll = -logp.gather(1, tgt[:, None])[:, 0]
    ref_loss = (1 - ls) * nll - ls * logp.mean(-1)
    ref_z = zw * lse ** 2
    (ref_loss + ref_z).mean().backward()
    loss = torch.empty(rows, device="cuda")
    z = torch.empty(rows, device="cuda")
    l2 = logits.clone()
    _ext().cross_entropy(l2, tgt, loss, z, None, ls, zw, 0.0, 1.0 / rows, True)
    assert torch.allclose(loss, ref_loss + ref_z, rtol=1e-3, atol=1e-3)
    assert torch.allclose(z, ref_z, rtol=1e-3, atol=1e-4)
    assert _rel_err(l2, lf.grad) < 2e-2


def test_embedding_fwd_bwd():
    torch.manual_seed(0)
    V, D, T = 1000, 256, 4096
    table = torch.randn(V, D, device="cuda", dtype=torch.bfloat16)
    ids = torch.randint(0, V, (T,), device="cuda")
    out = torch.empty(T, D, device="cuda", dtype=torch.bfloat16)
    e = _ext()
    e.embedding_fwd(table, ids, out, 1.0)
    assert torch.equal(out, table[ids])
    dout = torch.randn(T, D, device="cuda", dtype=torch.bfloat16)
    dt = torch.zeros(V, D, device="cuda")
    e.embedding_bwd(dout, ids, dt, 1.0)
    ref = torch.zeros(V, D, device="cuda").index_add_(0, ids, dout.float())
    assert _rel_err(dt, ref) < 1e-5


def test_adamw_and_sumsq():
    torch.manual_seed(0)
    n = 100003
    p = torch.randn(n, device="cuda")
    g = torch.randn(n, device="cuda")
    m = torch.zeros(n, device="cuda")
    v = torch.zeros(n, device="cuda")
    pb = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    ref_p = p.clone()
    lr, b1, b2, eps, wd = 1e-2, 0.9, 0.95, 1e-8, 0.1
    e = _ext()
    rm = torch.zeros(n, device="cuda")
    rv = torch.zeros(n, device="cuda")
    for t in range(1, 4):
        e.adamw_step(p, m, v, g, pb, lr, b1, b2, eps, wd, 1 - b1 ** t, 1 - b2 ** t, 1.0, None)
        rm = b1 * rm + (1 - b1) * g
        rv = b2 * rv + (1 - b2) * g * g
        ref_p = ref_p - lr * ((rm / (1 - b1 ** t)) / ((rv / (1 - b2 ** t)).sqrt() + eps) + wd * ref_p)
    assert torch.allclose(p, ref_p, rtol=1e-4, atol=1e-5)
    assert torch.equal(pb, p.bfloat16())
    out = torch.zeros(1, device="cuda")
    e.sumsq(g, out)
    assert torch.allclose(out[0], (g * g).sum(), rtol=1e-3)


@pytest.mark.parametrize("M,N,K", [(256, 512, 256), (384, 272, 1040), (128, 4096, 2048)])
def test_fp8_gemm_matches_dequantised_reference(M, N, K):
    """Per-tensor-scaled FP8 GEMM (e4m3 activations, e5m2 weights) against the fp32 product of the same quantised
    values; forward and the FP8 data gradient."""
    from mintext_b200.modules.linear import fp8_matmul_reference
    from mintext_b200.ops import functional as F
    from mintext_b200.ops._ext import check_status

    torch.manual_seed(0)
    x = torch.randn(M, K, device="cuda").bfloat16().requires_grad_(True)
    w = (torch.randn(K, N, device="cuda") * 0.05).bfloat16().requires_grad_(True)
    y = F.linear_fp8(x, w)
    ref = fp8_matmul_reference(x.detach(), w.detach(), torch.float32)
    torch.cuda.synchronize()
    check_status()
    rel = ((y.float() - ref).norm() / ref.norm()).item()
    assert rel < 1e-2, rel
    full = x.detach().float() @ w.detach().float()
    corr = torch.corrcoef(torch.stack([y.float().flatten(), full.flatten()]))[0, 1].item()
    assert corr > 0.99, corr
    dy = torch.randn_like(y)
    y.backward(dy)
    torch.cuda.synchronize()
    check_status()
    dx_ref = dy.float() @ w.detach().float().t()
    dw_ref = x.detach().float().t() @ dy.float()
    assert ((x.grad.float() - dx_ref).norm() / dx_ref.norm()).item() < 0.15   # two e5m2 operands
    assert ((w.grad.float() - dw_ref).norm() / dw_ref.norm()).item() < 1e-2


def _mx_dequant(q, sf, tile_rows):
    """Decode e4m3 elements and their UE8M0 block scales (512-byte atoms of 32 lanes x 16 bytes per 128 rows of a
    tile and 128-element k-block, tile-relative rows)."""
    R, K = q.shape
    atoms = (tile_rows + 127) // 128
    rows = torch.arange(R, device=q.device)[:, None]
    g = torch.arange(K // 32, device=q.device)[None, :]
    tile, rr = rows // tile_rows, rows % tile_rows
    off = ((tile * (K // 128) + (g >> 2)) * atoms + (rr >> 7)) * 512 + (rr & 31) * 16 + ((rr & 127) >> 5) * 4 + (g & 3)
    scale = torch.exp2(sf[off].float() - 127.0)
    return (q.view(torch.float8_e4m3fn).float().view(R, K // 32, 32) * scale[:, :, None]).view(R, K)


def test_mxfp8_quantise_blocks_and_transposed_copy():
    from mintext_b200.ops._ext import ext

    torch.manual_seed(0)
    x = (torch.randn(384, 512, device="cuda") * torch.logspace(-3, 2, 512, device="cuda")).bfloat16()
    q, sf, qt, sft = ext().mxfp8_quantize(x, True, False, True, True)
    xd = _mx_dequant(q, sf, 128)
    assert ((xd - x.float()).norm() / x.float().norm()).item() < 0.04
    # every block uses the e4m3 range: the largest magnitude of a block lands in (224, 448] after scaling
    blk = x.float().view(384, 16, 32).abs().amax(-1)
    qmax = q.view(torch.float8_e4m3fn).float().abs().view(384, 16, 32).amax(-1)
    assert (qmax[blk > 0] > 223).all() and (qmax <= 448).all()
    # the transposed copy equals quantising x^T along its rows
    q2, sf2, _, _ = ext().mxfp8_quantize(x.t().contiguous(), True, True, False, False)
    assert torch.equal(qt, q2) and torch.equal(sft, sf2)
    assert torch.allclose(_mx_dequant(qt, sft, 192), _mx_dequant(q2, sf2, 192))


@pytest.mark.parametrize("M,N,K", [(128, 192, 128), (384, 1000, 512), (1024, 2048, 2048), (2000, 776, 384)])
def test_mxfp8_gemm_matches_dequantised_reference(M, N, K):
    """Block-scaled FP8 GEMM against the fp32 product of the same de-quantised operands."""
    from mintext_b200.ops._ext import check_status, ext, status_word

    torch.manual_seed(0)
    x = (torch.randn(M, K, device="cuda") * torch.logspace(-2, 1, K, device="cuda")).bfloat16()
    w = (torch.randn(N, K, device="cuda") * 0.05).bfloat16()
    e = ext()
    xq, xs, _, _ = e.mxfp8_quantize(x, True, False, False, False)
    wq, ws, _, _ = e.mxfp8_quantize(w, True, True, False, False)
    y = e.gemm_mxfp8(xq, xs, wq, ws, status_word(x.device))
    torch.cuda.synchronize()
    check_status()
    ref = _mx_dequant(xq, xs, 128) @ _mx_dequant(wq, ws, 192).t()
    rel = ((y.float() - ref).norm() / ref.norm()).item()
    assert rel < 1e-2, rel
    full = x.float() @ w.float().t()
    assert ((y.float() - full).norm() / full.norm()).item() < 0.06


def test_mxfp8_linear_forward_and_gradients():
    from mintext_b200.ops import functional as F
    from mintext_b200.ops._ext import check_status

    torch.manual_seed(0)
    x = torch.randn(512, 384, device="cuda").bfloat16().requires_grad_(True)
    w = (torch.randn(384, 640, device="cuda") * 0.05).bfloat16().requires_grad_(True)
    assert F.mxfp8_kernel_path(x, w)
    y = F.linear_mxfp8(x, w)
    dy = torch.randn_like(y)
    y.backward(dy)
    torch.cuda.synchronize()
    check_status()
    full = x.detach().float() @ w.detach().float()
    assert ((y.float() - full).norm() / full.norm()).item() < 0.06
    dx_ref = dy.float() @ w.detach().float().t()
    dw_ref = x.detach().float().t() @ dy.float()
    assert ((x.grad.float() - dx_ref).norm() / dx_ref.norm()).item() < 0.06
    assert ((w.grad.float() - dw_ref).norm() / dw_ref.norm()).item() < 1e-2


def test_fp8_gated_mlp_front_half_matches_bf16_path():
    """One FP8 GEMM for gate|up plus the activation kernel, against the bf16 kernels (values and gradients)."""
    from mintext_b200.ops import functional as F
    from mintext_b200.ops._ext import check_status

    torch.manual_seed(5)
    T, K, M = 512, 256, 384
    x = torch.randn(T, K, device="cuda").bfloat16().requires_grad_(True)
    wg = (torch.randn(K, M, device="cuda") * 0.06).bfloat16().requires_grad_(True)
    wu = (torch.randn(K, M, device="cuda") * 0.06).bfloat16().requires_grad_(True)
    h8 = F.gate_up_act_fp8(x, wg, wu, "silu")
    g = torch.randn_like(h8)
    h8.backward(g)
    got = [h8.detach(), x.grad.clone(), wg.grad.clone(), wu.grad.clone()]
    x.grad = wg.grad = wu.grad = None
    h16 = F.gate_up_act(x, wg, wu, "silu")
    h16.backward(g)
    torch.cuda.synchronize()
    check_status()
    ref = [h16.detach(), x.grad, wg.grad, wu.grad]
    # e5m2 weights keep two mantissa bits: the comparison is against the bf16 path, not against an exact FP8 oracle
    for name, a, b, tol in zip(("h", "dx", "dwg", "dwu"), got, ref, (0.12, 0.25, 0.12, 0.12)):
        assert _rel_err(a, b) < tol, (name, _rel_err(a, b))


def test_mxfp8_mlp_matches_bf16_mlp():
    """The MLP with ``fp8_recipe=mx_block`` (one block-scaled GEMM for gate|up, block-scaled down projection and
    data gradients) against the same module on the bf16 kernels."""
    from mintext_b200 import MinTextConfig
    from mintext_b200.modules.linear import MLP
    from mintext_b200.ops._ext import check_status

    def build(**kw):
        c = MinTextConfig(hidden_size=256, intermediate_size=512, dtype="bfloat16", weight_dtype="bfloat16", **kw)
        return MLP(c, rngs=torch.Generator().manual_seed(3)).cuda()

    torch.manual_seed(1)
    x = torch.randn(4, 128, 256, device="cuda").bfloat16()
    outs = []
    for kw in ({}, {"use_fp8": True, "fp8_recipe": "mx_block"}):
        m = build(**kw)
        xi = x.clone().requires_grad_(True)
        y = m(xi)
        y.backward(torch.ones_like(y) * 0.01)
        outs.append((y.detach(), xi.grad, m.gate.kernel.grad, m.down.kernel.grad))
    torch.cuda.synchronize()
    check_status()
    for name, a, b in zip(("y", "dx", "dw_gate", "dw_down"), outs[1], outs[0]):
        assert a is not None and _rel_err(a, b) < 0.08, (name, _rel_err(a, b))


@pytest.mark.parametrize("kind", ["sigmoid", "silu"])
def test_gate_mul_matches_torch_with_strided_gate(kind):
    """x * f(gate) with the gate a column block of a wider projection (no copy), values and both gradients."""
    from mintext_b200.ops import functional as F
    from mintext_b200.ops._ext import check_status

    torch.manual_seed(0)
    B, S, H, dh = 2, 96, 4, 64
    proj = torch.randn(B, S, H, 2 * dh, device="cuda").bfloat16().requires_grad_(True)
    x = torch.randn(B, S, H, dh, device="cuda").bfloat16().requires_grad_(True)
    _, gate = proj.chunk(2, dim=-1)
    y = F.gate_mul(x, gate, kind)
    dy = torch.randn_like(y)
    y.backward(dy)
    torch.cuda.synchronize()
    check_status()
    xf, pf = x.detach().float().requires_grad_(True), proj.detach().float().requires_grad_(True)
    gf = pf.chunk(2, dim=-1)[1]
    ref = xf * (torch.sigmoid(gf) if kind == "sigmoid" else torch.nn.functional.silu(gf))
    ref.backward(dy.float())
    assert _rel_err(y, ref) < 1e-2
    assert _rel_err(x.grad, xf.grad) < 1e-2
    assert _rel_err(proj.grad[..., dh:], pf.grad[..., dh:]) < 1e-2
    assert proj.grad[..., :dh].abs().max() == 0



@pytest.mark.parametrize("T,K,I,act", [(384, 256, 256, "silu"), (1000, 192, 128, "gelu_pytorch_tanh"), (2048, 512, 1024, "silu")])
def test_fused_gate_up_act_gemm_matches_separate_kernels(T, K, I, act, monkeypatch):
    """One CTA-pair GEMM producing [gate | up] and act(gate) * up from its epilogue, against the two GEMMs plus the
    activation kernel (values of both outputs, and the gradients that flow through either path)."""
    from mintext_b200.ops import functional as F
    from mintext_b200.ops._ext import check_status

    torch.manual_seed(2)
    x = torch.randn(T, K, device="cuda").bfloat16()
    wg = (torch.randn(K, I, device="cuda") * K ** -0.5).bfloat16()
    wu = (torch.randn(K, I, device="cuda") * K ** -0.5).bfloat16()
    dy = torch.randn(T, I, device="cuda").bfloat16()
    res = {}
    for mode in ("1", "0"):
        monkeypatch.setenv("MT_FUSED_GATE_UP", mode)
        xi, g, u = (t.clone().requires_grad_(True) for t in (x, wg, wu))
        h = F.gate_up_act(xi, g, u, act)
        h.backward(dy)
        res[mode] = (h.detach(), xi.grad, g.grad, u.grad)
    torch.cuda.synchronize()
    check_status()
    ref = oracle_h = None
    xf = x.float()
    gf, uf = xf @ wg.float(), xf @ wu.float()
    from mintext_b200.ops import oracle
    oracle_h = oracle.activation(act)(gf) * uf
    assert _rel_err(res["1"][0], oracle_h) < 1e-2
    for name, a, b in zip(("h", "dx", "dwg", "dwu"), res["1"], res["0"]):
        assert _rel_err(a, b) < 1e-2, (name, _rel_err(a, b))


@pytest.mark.parametrize("T,D,I,act", [(512, 256, 512, "silu"), (1000, 192, 256, "gelu_pytorch_tanh"), (2048, 512, 1024, "silu")])
def test_gated_mlp_single_node_matches_separate_kernels(T, D, I, act, monkeypatch):
    """The whole gated MLP as one autograd node (fused gate/up GEMM forward; down-projection data gradient with the
    activation backward in its epilogue) against the chain of separate GEMMs and activation kernels."""
    from mintext_b200.ops import functional as F
    from mintext_b200.ops._ext import check_status

    torch.manual_seed(4)
    x = torch.randn(T, D, device="cuda").bfloat16()
    wg = (torch.randn(D, I, device="cuda") * D ** -0.5).bfloat16()
    wu = (torch.randn(D, I, device="cuda") * D ** -0.5).bfloat16()
    wd = (torch.randn(I, D, device="cuda") * I ** -0.5).bfloat16()
    dy = torch.randn(T, D, device="cuda").bfloat16()
    res = {}
    for mode in ("1", "0"):
        monkeypatch.setenv("MT_FUSED_GATE_UP", mode)
        xi, g, u, d = (t.clone().requires_grad_(True) for t in (x, wg, wu, wd))
        assert F.gated_mlp_path(xi, g, u, d, act) == (mode == "1")
        y = F.gated_mlp(xi, g, u, d, act) if mode == "1" else F.linear(F.gate_up_act(xi, g, u, act), d)
        y.backward(dy)
        res[mode] = (y.detach(), xi.grad, g.grad, u.grad, d.grad)
    torch.cuda.synchronize()
    check_status()
    for name, a, b in zip(("y", "dx", "dwg", "dwu", "dwd"), res["1"], res["0"]):
        assert _rel_err(a, b) < 1.5e-2, (name, _rel_err(a, b))


def test_threefry_randint_kernel_equals_the_tensor_path():
    from mintext_b200.utils import threefry as tf

    for seed, (row_lo, rows, cols, span) in enumerate([(0, 4, 128, 128256), (5, 3, 100, 17), (2 ** 20, 2, 4096, 151936)]):
        k = tf.key(seed + 11)
        got = tf.randint_rows(k, row_lo, rows, cols, span, device="cuda", use_kernel=True)
        want = tf.randint_rows(k, row_lo, rows, cols, span, device="cpu", use_kernel=False)
        assert got.dtype == torch.int64 and torch.equal(got.cpu(), want)


def test_gate_up_mxfp8_matches_the_concatenated_linear_and_reuses_quantised_weights():
    """One block-scaled GEMM for [gate | up]: same values as the block-scaled linear on the concatenated weight, weight
    gradients added straight into each parameter's fp32 accumulator, and the quantised weight copy kept until the
    parameters are declared changed."""
    from mintext_b200.ops import functional as F

    torch.manual_seed(11)
    T, K, M = 256, 256, 384
    x = (torch.randn(T, K, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_(True)
    wg = (torch.randn(K, M, device="cuda") * 0.05).to(torch.bfloat16).requires_grad_(True)
    wu = (torch.randn(K, M, device="cuda") * 0.05).to(torch.bfloat16).requires_grad_(True)
    wg.main_grad = torch.zeros(K, M, device="cuda")
    wu.main_grad = torch.zeros(K, M, device="cuda")
    cache = F.QuantisedWeightCache()
    y = F.gate_up_mxfp8(x, wg, wu, cache)
    first = cache.entry
    x2 = x.detach().clone().requires_grad_(True)
    wcat = torch.cat([wg.detach(), wu.detach()], dim=1).requires_grad_(True)
    ref = F.linear_mxfp8(x2, wcat)
    assert torch.equal(y, ref)
    dy = torch.randn_like(y)
    y.backward(dy)
    ref.backward(dy)
    _check()
    assert torch.equal(x.grad, x2.grad)
    assert wg.grad is None and wu.grad is None
    assert _rel_err(wg.main_grad, wcat.grad[:, :M].float()) < 1e-2
    assert _rel_err(wu.main_grad, wcat.grad[:, M:].float()) < 1e-2
    F.gate_up_mxfp8(x, wg, wu, cache)
    assert cache.entry is first          # same parameters: no second quantisation
    F.bump_weight_version()
    F.gate_up_mxfp8(x, wg, wu, cache)
    assert cache.entry is not first      # the optimizer has stepped: quantised again


def test_adamw_tracks_a_float64_reference_over_many_steps():
    """The fused AdamW against the same recurrence in float64, 50 steps with gradients spanning ten orders of
    magnitude: parameters and both moments stay within fp32 rounding of the exact recurrence (errors measured against
    each element's gradient scale, since a moment that cancels to near zero has no meaningful relative error)."""
    torch.manual_seed(1)
    n = 65536 + 5
    e = _ext()
    p = torch.randn(n, device="cuda")
    m = torch.zeros(n, device="cuda")
    v = torch.zeros(n, device="cuda")
    scale = 10.0 ** torch.randint(-8, 2, (n,), device="cuda").float()
    rp, rm, rv = p.double(), m.double(), v.double()
    lr, b1, b2, eps, wd = 3e-3, 0.9, 0.95, 1e-8, 0.1
    for t in range(1, 51):
        g = torch.randn(n, device="cuda") * scale
        e.adamw_step(p, m, v, g, None, lr, b1, b2, eps, wd, 1 - b1 ** t, 1 - b2 ** t, 1.0, None)
        gd = g.double()
        rm = b1 * rm + (1 - b1) * gd
        rv = b2 * rv + (1 - b2) * gd * gd
        rp = rp - lr * ((rm / (1 - b1 ** t)) / ((rv / (1 - b2 ** t)).sqrt() + eps) + wd * rp)
    _check()
    sd = scale.double()
    assert float((p.double() - rp).abs().max()) < 2e-5
    assert float(((m.double() - rm).abs() / sd).max()) < 1e-5
    assert float(((v.double() - rv).abs() / (sd * sd)).max()) < 1e-5
