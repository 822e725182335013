"""Muon's Newton-Schulz orthogonalisation on the tcgen05 GEMM kernel (bf16 operands, fp32 accumulation).

Per iteration three GEMMs of this repository's dense kernel: ``A = X X^T``, ``A2 = A A`` and
``X <- a X + (b A + c A2) X`` (the last one accumulates into an fp32 copy of ``a X`` through the kernel's TMA-add
epilogue).  Semantics follow ``optax.contrib.muon`` as used by the reference (mintext/optim/optimizer.py:117-168):
wide orientation, Frobenius normalisation, coefficients (3.4445, -4.7750, 2.0315).
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
    for i in range(bsz):
        m = x[i]
        transposed = r > c
        if transposed:
            m = m.t()
        m = m / (m.norm() + eps)
        X = m.to(torch.bfloat16).contiguous()
        n = X.shape[0]
        Xf = None
        for _ in range(steps):
            A = _gemm(X, X, torch.empty(n, n, device=x.device, dtype=torch.bfloat16), False, False)   # X X^T
            A2 = _gemm(A, A, torch.empty_like(A), False, True)                                         # A A
            Bm = A.float().mul_(cb).add_(A2.float(), alpha=cc).to(torch.bfloat16)
            Xf = X.float().mul_(ca)
            _gemm(Bm, X, Xf, False, True, accumulate=True)                                             # += B X
            X = Xf.to(torch.bfloat16)
        out[i] = Xf.t() if transposed else Xf
    return out
