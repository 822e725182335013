"""Muon's Newton-Schulz orthogonalisation on the tcgen05 GEMM kernel (bf16 operands, fp32 accumulation).

Per iteration three GEMMs of this repository's dense kernel and three scalings, everything in bf16 between the GEMMs:
``A = X X^T``; ``B = b A`` prefilled and ``(c A) A`` added into it by the kernel's TMA-add epilogue; ``X' = a X``
prefilled and ``B X`` added into it.  No fp32 <-> bf16 cast passes; only the last iteration accumulates into an fp32
copy of ``a X`` so that the returned update keeps the accumulator's precision.  Semantics follow
``optax.contrib.muon`` as used by the reference (mintext/optim/optimizer.py:117-168): wide orientation, Frobenius
normalisation, coefficients (3.4445, -4.7750, 2.0315).
"""

from __future__ import annotations

import torch

from . import oracle
from ._ext import ext, status_word


def _gemm(a, b, c, a_km, b_kn, accumulate=False):
    ext().gemm(a, b, c, a_km, b_kn, accumulate, status_word(a.device))
    return c


def kernel_path(rows: int, cols: int, x: torch.Tensor) -> bool:
    return x.is_cuda and rows % 8 == 0 and cols % 8 == 0 and min(rows, cols) >= 64 and hasattr(ext(), "gemm")


def newton_schulz(x: torch.Tensor, steps: int = 5, eps: float = 1e-8, coeffs=oracle.NS_COEFFS) -> torch.Tensor:
    """``x [batch, rows, cols]`` fp32 -> orthogonalised fp32 of the same shape."""
    bsz, r, c = x.shape
    if not kernel_path(r, c, x):
        return oracle.newton_schulz(x, steps, eps, coeffs)
    ca, cb, cc = coeffs
    out = torch.empty_like(x)
    bf = torch.bfloat16
    for i in range(bsz):
        m = x[i]
        transposed = r > c
        if transposed:
            m = m.t()
        m = m / (m.norm() + eps)
        X = m.to(bf).contiguous()
        n, w = X.shape
        A, Ac, Bm = (torch.empty(n, n, device=x.device, dtype=bf) for _ in range(3))
        Xn = torch.empty(n, w, device=x.device, dtype=bf)
        Xf = None
        for it in range(steps):
            _gemm(X, X, A, False, False)                         # A = X X^T
            torch.mul(A, cb, out=Bm)
            torch.mul(A, cc, out=Ac)
            _gemm(Ac, A, Bm, False, True, accumulate=True)       # B = b A + (c A) A
            if it == steps - 1:
                Xf = X.float().mul_(ca)
                _gemm(Bm, X, Xf, False, True, accumulate=True)   # fp32: a X + B X
            else:
                torch.mul(X, ca, out=Xn)
                _gemm(Bm, X, Xn, False, True, accumulate=True)   # X' = a X + B X
                X, Xn = Xn, X
        if Xf is None:
            Xf = X.float()
        out[i] = Xf.t() if transposed else Xf
    return out
