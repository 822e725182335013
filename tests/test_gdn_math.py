"""The algebra the chunk-parallel Gated Delta Rule kernels implement (csrc/gdn/gdn_prep.cu), restated with plain tensor
operations and checked on the CPU: the blocked inverse of the unit lower-triangular WY matrix, and the hand-derived
backward pass (operand gradients -> input gradients) against autograd of the batched tensor-algebra form."""

import pytest
import torch

from mintext_b200.ops.gdn import prep_torch

L = 64


def blocked_inverse(A: torch.Tensor) -> torch.Tensor:
    """``(I - A)^-1`` for strictly lower-triangular ``A [N, 64, 64]`` the way the kernel does it: the four 16x16
    diagonal blocks by forward substitution, then block row ``b`` from the rows above it,
    ``T[b, :b] = D_b (A[b, :b] T[:b, :b])``."""
    N = A.shape[0]
    T = torch.zeros_like(A)
    D = []
    for b in range(4):
        Abb = A[:, 16 * b:16 * b + 16, 16 * b:16 * b + 16]
        Db = torch.zeros_like(Abb)
        for i in range(16):
            row = torch.zeros(N, 16, dtype=A.dtype)
            row[:, i] = 1
            for j in range(i):
                row = row + Abb[:, i, j, None] * Db[:, j, :]
            Db[:, i, :] = row
        D.append(Db)
    for b in range(4):
        T[:, 16 * b:16 * b + 16, 16 * b:16 * b + 16] = D[b]
        if b > 0:
            R = A[:, 16 * b:16 * b + 16, :16 * b] @ T[:, :16 * b, :16 * b]
            T[:, 16 * b:16 * b + 16, :16 * b] = D[b] @ R
    return T


def analytic_backward(q, k, v, beta, g, T, dW, dU, dQG, dM, dKD, dGL):
    """Input gradients from operand gradients, phase by phase as in ``gdn_prep_bwd_kernel``."""
    dk_dim = q.shape[-1]
    s = dk_dim ** -0.5
    rq = torch.rsqrt((q * q).sum(-1, keepdim=True) + 1e-6)
    rk = torch.rsqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    qn, kn = q * rq * s, k * rk
    G = g.cumsum(-1)
    eG = torch.exp(G.clamp(-30, 30))
    mG = ((G > -30) & (G < 30)).to(q.dtype)
    diff = G[..., :, None] - G[..., None, :]
    tril = torch.tril(torch.ones(L, L, dtype=q.dtype))
    stril = torch.tril(torch.ones(L, L, dtype=q.dtype), -1)
    decay = torch.exp(diff.clamp(-30, 30)) * tril
    md = ((diff > -30) & (diff < 30)).to(q.dtype)
    dl = G[..., -1:] - G
    eKD = torch.exp(dl.clamp(-30, 30))
    mKD = ((dl > -30) & (dl < 30)).to(q.dtype)
    Tt = T.transpose(-1, -2)
    # phases A, B: through U = T (beta v) and W = T (beta e^G kn)
    dT = dU @ (v * beta[..., None]).transpose(-1, -2) + dW @ (kn * (beta * eG)[..., None]).transpose(-1, -2)
    dBV, dBK = Tt @ dU, Tt @ dW
    # phase C: through T = (I - A)^-1
    dA = (Tt @ dT @ Tt) * stril
    # phase D: through A and M to the Gram matrices, beta and the decays
    P, QK = kn @ kn.transpose(-1, -2), qn @ kn.transpose(-1, -2)
    dP = -beta[..., None] * decay * dA
    dMm = dM * tril
    dQK = dMm * decay
    E = (-beta[..., None] * P * dA + dMm * QK) * decay * md
    dG = E.sum(-1) - E.sum(-2)
    sBK = (dBK * kn).sum(-1) * eG
    dbeta = (-P * decay * dA).sum(-1) + (dBV * v).sum(-1) + sBK
    # phase E: normalised queries / keys, then the normalisations
    dqn = dQK @ kn + dQG * eG[..., None]
    dkn = dQK.transpose(-1, -2) @ qn + (dP + dP.transpose(-1, -2)) @ kn + dBK * (beta * eG)[..., None] + dKD * eKD[..., None]
    sKD = (dKD * kn).sum(-1) * eKD * mKD
    dG = dG + ((dQG * qn).sum(-1) * eG + beta * sBK) * mG - sKD
    dG[..., -1] += sKD.sum(-1) + dGL * eG[..., -1] * mG[..., -1]
    # phase F: the cumulative sum's gradient is a reverse cumulative sum
    dg = dG.flip(-1).cumsum(-1).flip(-1)
    dv = dBV * beta[..., None]
    dq = s * rq * dqn - s * rq ** 3 * q * (q * dqn).sum(-1, keepdim=True)
    dk = rk * dkn - rk ** 3 * k * (k * dkn).sum(-1, keepdim=True)
    return dq, dk, dv, dbeta, dg


def _inputs(N, dk, dv, decay_scale, seed):
    g = torch.Generator().manual_seed(seed)
    mk = lambda *s: torch.randn(*s, generator=g, dtype=torch.float64)
    q, k, v = mk(1, N, L, dk), mk(1, N, L, dk), mk(1, N, L, dv)
    beta = torch.rand(1, N, L, generator=g, dtype=torch.float64)
    gl = -torch.rand(1, N, L, generator=g, dtype=torch.float64) * decay_scale
    return [t.reshape(1, N, L, -1).squeeze(-1) if t.dim() == 3 else t for t in (q, k, v, beta, gl)]


@pytest.mark.parametrize("seed", [0, 1])
def test_blocked_inverse_equals_the_triangular_solve(seed):
    g = torch.Generator().manual_seed(seed)
    A = torch.tril(torch.randn(3, L, L, generator=g, dtype=torch.float64) * 0.3, -1)
    eye = torch.eye(L, dtype=torch.float64)
    want = torch.linalg.solve_triangular(eye - A, eye.expand_as(A).contiguous(), upper=False)
    assert torch.allclose(blocked_inverse(A), want, atol=1e-10)


@pytest.mark.parametrize("dk,dv,decay_scale", [(16, 8, 0.5), (32, 32, 0.05), (16, 16, 3.0)])
def test_analytic_backward_equals_autograd(dk, dv, decay_scale):
    """``decay_scale = 3`` drives the cumulative log-decay past the -30 clamp inside a chunk."""
    q, k, v, beta, g = _inputs(3, dk, dv, decay_scale, seed=2)
    # prep_torch takes [B, H, S, d]: one batch, three heads of one chunk each
    ins = [t.clone().requires_grad_(True) for t in (q, k, v, beta, g)]
    outs = prep_torch(*ins)
    gen = torch.Generator().manual_seed(9)
    cots = [torch.randn(o.shape, generator=gen, dtype=torch.float64) for o in outs]
    want = torch.autograd.grad(outs, ins, cots)
    with torch.no_grad():
        kn = k * torch.rsqrt((k * k).sum(-1, keepdim=True) + 1e-6)
        G = g.cumsum(-1)
        decay = torch.exp((G[..., :, None] - G[..., None, :]).clamp(-30, 30))
        A = (-(kn * beta[..., None]) @ kn.transpose(-1, -2) * decay) * torch.tril(torch.ones(L, L, dtype=torch.float64), -1)
        T = blocked_inverse(A[0])[None]
        # operands come back as [B*H, C=1, 64, ...]: back to [1, H, 64, ...]
        dW, dU, dQG, dM, dKD, dGL = (c.reshape(1, 3, *c.shape[2:]) if c.dim() == 4 else c.reshape(1, 3) for c in cots)
        got = analytic_backward(q, k, v, beta, g, T, dW, dU, dQG, dM, dKD, dGL)
    for name, a, b in zip("q k v beta g".split(), got, want):  # the tensor-algebra form computes in fp32
        assert torch.allclose(a, b.double(), atol=2e-5, rtol=1e-4), (name, float((a - b).abs().max()))
