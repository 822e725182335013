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
