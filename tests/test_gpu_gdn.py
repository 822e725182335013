"""Gated Delta Rule state-recurrence kernels (forward and backward) against the plain PyTorch formulation."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


def _py_scan(W, U, QG, M, KD, GL):
    BH, C, L, dk = W.shape
    S = torch.zeros(BH, dk, U.shape[-1], device=W.device)
    out = []
    for c in range(C):
        Vp = U[:, c] - W[:, c] @ S
        out.append(QG[:, c] @ S + M[:, c] @ Vp)
        S = GL[:, c, None, None] * S + KD[:, c].transpose(-1, -2) @ Vp
    return torch.stack(out, 1)


@pytest.mark.parametrize("dk,dv,C", [(64, 64, 3), (128, 128, 5), (64, 96, 1)])
def test_scan_kernel_forward_and_all_gradients(dk, dv, C):
    from mintext_b200.ops.gdn import _ScanFn

    torch.manual_seed(0)
    BH, L = 3, 64
    mk = lambda *s, sc=1.0: (torch.randn(*s, device="cuda") * sc).requires_grad_(True)
    W, QG, KD = mk(BH, C, L, dk, sc=0.1), mk(BH, C, L, dk, sc=0.1), mk(BH, C, L, dk, sc=0.1)
    U, M = mk(BH, C, L, dv), mk(BH, C, L, L, sc=0.1)
    GL = torch.rand(BH, C, device="cuda").requires_grad_(True)
    ins = (W, U, QG, M, KD, GL)
    out = _ScanFn.apply(*ins)
    ref_ins = [t.detach().clone().requires_grad_(True) for t in ins]
    ref = _py_scan(*ref_ins)
    assert _rel(out, ref) < 1e-5, _rel(out, ref)
    g = torch.randn_like(out)
    out.backward(g)
    ref.backward(g)
    for name, a, b in zip("W U QG M KD GL".split(), ins, ref_ins):
        if b.grad is None:  # a single chunk: the state update after it reaches no output
            assert float(a.grad.abs().max()) == 0.0, name
        else:
            assert _rel(a.grad, b.grad) < 1e-4, (name, _rel(a.grad, b.grad))


@pytest.mark.parametrize("dk,dv,S", [(64, 64, 200), (128, 128, 256)])
def test_chunk_gated_delta_rule_kernel_path_matches_oracle(dk, dv, S):
    from mintext_b200.ops import oracle
    from mintext_b200.ops.gdn import chunk_gated_delta_rule_cuda, cuda_path

    torch.manual_seed(1)
    B, H = 2, 3
    q, k = torch.randn(B, H, S, dk, device="cuda"), torch.randn(B, H, S, dk, device="cuda")
    v = torch.randn(B, H, S, dv, device="cuda")
    beta = torch.rand(B, H, S, device="cuda")
    g = -torch.rand(B, H, S, device="cuda") * 0.5
    assert cuda_path(q, v)
    ins = [t.requires_grad_(True) for t in (q, k, v, beta, g)]
    out = chunk_gated_delta_rule_cuda(*ins)
    ref_ins = [t.detach().clone().requires_grad_(True) for t in ins]
    ref = oracle.chunk_gated_delta_rule(*ref_ins)
    assert _rel(out, ref) < 1e-4
    go = torch.randn_like(out)
    out.backward(go)
    ref.backward(go)
    for name, a, b in zip("q k v beta g".split(), ins, ref_ins):
        assert _rel(a.grad, b.grad) < 2e-3, (name, _rel(a.grad, b.grad))


@pytest.mark.parametrize("dk,dv,S", [(64, 64, 128), (128, 128, 200), (64, 96, 70), (128, 32, 64)])
def test_prep_kernel_operands_and_gradients_match_tensor_algebra(dk, dv, S):
    """The chunk-parallel kernels against the batched tensor-algebra form: every scan operand, then the gradients of
    random cotangents on all of them, with token-major (strided) inputs and a ragged last chunk."""
    from mintext_b200.ops.gdn import _PrepFn, prep_kernel_path, prep_torch

    torch.manual_seed(2)
    B, H = 2, 3
    assert prep_kernel_path(dk, dv)
    mk = lambda *s: torch.randn(*s, device="cuda")
    # [B, S, H, d] storage seen as [B, H, S, d], as the layer hands it over
    q, k, v = mk(B, S, H, dk).transpose(1, 2), mk(B, S, H, dk).transpose(1, 2), mk(B, S, H, dv).transpose(1, 2)
    beta = torch.rand(B, S, H, device="cuda").transpose(1, 2)
    g = (-torch.rand(B, S, H, device="cuda") * 0.5).transpose(1, 2)
    ins = [t.detach().clone(memory_format=torch.preserve_format).requires_grad_(True) for t in (q, k, v, beta, g)]
    assert not ins[0].is_contiguous()
    ref_ins = [t.detach().clone().requires_grad_(True) for t in (q, k, v, beta, g)]
    outs = _PrepFn.apply(*ins)
    refs = prep_torch(*ref_ins)
    names = "W U QG M KD GL".split()
    for n, a, b in zip(names, outs, refs):
        assert a.shape == b.shape, n
        assert _rel(a, b) < 2e-5, (n, _rel(a, b))
    cots = [torch.randn_like(o) for o in refs]
    torch.autograd.backward(outs, cots)
    torch.autograd.backward(refs, cots)
    for n, a, b in zip("q k v beta g".split(), ins, ref_ins):
        assert a.grad.shape == b.grad.shape, n
        assert _rel(a.grad, b.grad) < 2e-4, (n, _rel(a.grad, b.grad))


def test_prep_kernel_with_strong_decay_hits_the_clamp_like_the_tensor_form():
    """Log-decays large enough that ``G_i - G_j`` passes the -30 clamp inside a chunk."""
    from mintext_b200.ops.gdn import _PrepFn, prep_torch

    torch.manual_seed(3)
    B, H, S, d = 1, 2, 128, 64
    q, k, v = (torch.randn(B, H, S, d, device="cuda") for _ in range(3))
    beta = torch.rand(B, H, S, device="cuda")
    g = -torch.rand(B, H, S, device="cuda") * 2.0
    ins = [t.clone().requires_grad_(True) for t in (q, k, v, beta, g)]
    ref_ins = [t.clone().requires_grad_(True) for t in (q, k, v, beta, g)]
    outs, refs = _PrepFn.apply(*ins), prep_torch(*ref_ins)
    for a, b in zip(outs, refs):
        assert _rel(a, b) < 2e-5
    cots = [torch.randn_like(o) for o in refs]
    torch.autograd.backward(outs, cots)
    torch.autograd.backward(refs, cots)
    for n, a, b in zip("q k v beta g".split(), ins, ref_ins):
        assert _rel(a.grad, b.grad) < 2e-4, (n, _rel(a.grad, b.grad))
