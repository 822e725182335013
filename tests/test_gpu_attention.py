"""Flash attention kernels (tcgen05) against the fp32-softmax oracle, forward and backward."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


def _assert_blocks_close(got, ref, rel, what):
    """Per (batch, 128-token block, head) error: a single bad tile of one head must not hide in the global norm."""
    B, S, H, D = ref.shape
    nb = max(S // 128, 1)
    d = (got.float() - ref.float()).reshape(B, nb, S // nb, H, D).permute(0, 1, 3, 2, 4).reshape(B, nb, H, -1)
    r = ref.float().reshape(B, nb, S // nb, H, D).permute(0, 1, 3, 2, 4).reshape(B, nb, H, -1)
    err = d.norm(dim=-1) / (r.norm(dim=-1) + 1e-3 * r.norm() / (B * nb * H) ** 0.5 + 1e-12)
    assert err.max().item() < rel, (what, "worst block", err.max().item())


def _run(B, S, H, Hkv, d, causal=True, window=None, softcap=None, grad=True, dv=None):
    from mintext_b200.ops import oracle
    from mintext_b200.ops._ext import check_status
    from mintext_b200.ops.attention import flash_attention

    torch.manual_seed(0)
    q = torch.randn(B, S, H, d, device="cuda", dtype=torch.bfloat16, requires_grad=grad)
    k = torch.randn(B, S, Hkv, d, device="cuda", dtype=torch.bfloat16, requires_grad=grad)
    v = torch.randn(B, S, Hkv, dv or d, device="cuda", dtype=torch.bfloat16, requires_grad=grad)
    scale = d ** -0.5
    o = flash_attention(q, k, v, scale, causal, window, softcap)
    qf, kf, vf = (t.detach().float().requires_grad_(grad) for t in (q, k, v))
    ref = oracle.attention(qf, kf, vf, scale, causal, window, softcap)
    torch.cuda.synchronize()
    check_status()
    assert _rel(o, ref) < 2e-2, _rel(o, ref)
    _assert_blocks_close(o, ref, 4e-2, "o")
    if grad:
        do = torch.randn_like(o)
        o.backward(do)
        ref.backward(do.float())
        torch.cuda.synchronize()
        check_status()
        assert _rel(v.grad, vf.grad) < 3e-2, ("dv", _rel(v.grad, vf.grad))
        assert _rel(k.grad, kf.grad) < 3e-2, ("dk", _rel(k.grad, kf.grad))
        assert _rel(q.grad, qf.grad) < 3e-2, ("dq", _rel(q.grad, qf.grad))
        _assert_blocks_close(v.grad, vf.grad, 6e-2, "dv")
        _assert_blocks_close(k.grad, kf.grad, 6e-2, "dk")
        _assert_blocks_close(q.grad, qf.grad, 6e-2, "dq")


def test_flash_fwd_single_block():
    _run(1, 128, 1, 1, 64, grad=False)


def test_flash_fwd_multi_block_gqa():
    _run(2, 512, 4, 2, 64, grad=False)


def test_flash_fwd_dh128():
    _run(1, 384, 2, 1, 128, grad=False)


def test_flash_fwd_noncausal():
    _run(1, 256, 2, 2, 64, causal=False, grad=False)


def test_flash_bwd_single_block():
    _run(1, 128, 1, 1, 64)


def test_flash_bwd_multi_block_gqa():
    _run(2, 512, 4, 2, 64)


def test_flash_bwd_dh128():
    _run(1, 128, 1, 1, 128)
    _run(2, 512, 4, 2, 128)


def test_flash_bwd_dh128_window_and_softcap():
    _run(1, 512, 2, 1, 128, window=200)
    _run(1, 256, 2, 2, 128, softcap=30.0)
    _run(1, 256, 2, 1, 128, causal=False)


def test_flash_mla_shape_fwd():
    _run(1, 256, 2, 2, 192, grad=False, dv=128)
    _run(2, 512, 4, 4, 192, causal=False, grad=False, dv=128)


def test_flash_mla_shape_bwd():
    _run(1, 128, 1, 1, 192, dv=128)
    _run(2, 512, 4, 4, 192, dv=128)
    _run(1, 384, 2, 2, 192, causal=False, dv=128)


def test_flash_fwd_dh256():
    _run(1, 128, 1, 1, 256, grad=False)
    _run(2, 512, 4, 2, 256, grad=False)
    _run(1, 256, 2, 1, 256, causal=False, grad=False)


def test_flash_bwd_dh256():
    """head_dim 256 (Gemma 3) runs the backward as a dV pass and a dK / dQ pass."""
    _run(1, 128, 1, 1, 256)
    _run(2, 512, 4, 2, 256)
    _run(1, 512, 2, 1, 256, window=200)
    _run(1, 256, 2, 2, 256, softcap=30.0)
    _run(1, 256, 2, 1, 256, causal=False)


def test_flash_window_and_softcap():
    _run(1, 512, 2, 1, 64, window=200)
    _run(1, 256, 2, 2, 64, softcap=30.0)


def test_flash_strided_qkv_views():
    """q/k/v may be column blocks of one fused projection buffer."""
    from mintext_b200.ops import oracle
    from mintext_b200.ops.attention import flash_attention

    torch.manual_seed(1)
    B, S, H, Hkv, d = 1, 256, 4, 2, 64
    buf = torch.randn(B, S, (H + 2 * Hkv) * d, device="cuda", dtype=torch.bfloat16)
    q = buf[..., : H * d].view(B, S, H, d)
    k = buf[..., H * d:(H + Hkv) * d].view(B, S, Hkv, d)
    v = buf[..., (H + Hkv) * d:].view(B, S, Hkv, d)
    o = flash_attention(q, k, v, d ** -0.5)
    ref = oracle.attention(q.float(), k.float(), v.float(), d ** -0.5)
    assert _rel(o, ref) < 2e-2
