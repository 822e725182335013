"""CUDA path of the chunked Gated Delta Rule (reference: mintext/modules/linear_attention.py:49-205).

Two kernels each way.  The chunk-parallel part (L2 normalisation, decay matrices, the unit-lower-triangular WY
inverse, the per-chunk operands) is one CTA per (batch, head, chunk) working in shared memory
(``csrc/gdn/gdn_prep.cu``; its backward takes the operand gradients back to q, k, v, beta, g).  The sequential walk over
the chunks with the ``[dk, dv]`` state, which the plain implementation runs as a Python loop of small matmuls, is
``csrc/gdn/gdn_scan.cu``: the state slice of 32 value columns lives in shared memory for the whole sequence and the
per-chunk operands are staged once.  Value head dims above 128 keep the chunk-parallel part as batched tensor algebra
(``MT_GDN_PREP=torch`` selects that path everywhere).
"""

from __future__ import annotations

import os

import torch
import torch.nn.functional as TF

from . import functional as F
from . import oracle
from ._ext import ext

_L = 64


def cuda_path(q: torch.Tensor, v: torch.Tensor | None = None, chunk_size: int = _L) -> bool:
    if not (q.is_cuda and F._backend() != "oracle" and hasattr(ext(), "gdn_scan_fwd") and chunk_size == _L):
        return False
    dk = q.shape[-1]
    dv = v.shape[-1] if v is not None else dk
    return dk in (64, 128) and dv % 32 == 0


class _ScanFn(torch.autograd.Function):
    """``O`` of the recurrence ``V' = U - W S; O = QG S + M V'; S <- gl S + KD^T V'`` over the chunk axis."""

    @staticmethod
    def forward(ctx, W, U, QG, M, KD, GL):
        args = [t.contiguous() for t in (W, U, QG, M, KD, GL)]
        O, S = ext().gdn_scan_fwd(*args)
        ctx.save_for_backward(*args, S)
        return O

    @staticmethod
    def backward(ctx, dO):
        W, U, QG, M, KD, GL, S = ctx.saved_tensors
        dW, dU, dQG, dM, dKD, dGL = ext().gdn_scan_bwd(W, U, QG, M, KD, GL, S, dO.contiguous())
        return dW, dU, dQG, dM, dKD, dGL


def prep_kernel_path(dk: int, dv: int) -> bool:
    """True when the chunk-parallel stage runs as the ``gdn_prep`` kernels."""
    return (os.environ.get("MT_GDN_PREP", "kernel") != "torch" and hasattr(ext(), "gdn_prep_fwd")
            and dk in (64, 128) and dv % 32 == 0 and 0 < dv <= 128)


def _rows_ok(t: torch.Tensor) -> torch.Tensor:
    """The kernels read rows as 16-byte vectors through arbitrary batch / head / token strides."""
    if t.stride(-1) == 1 and all(s % 4 == 0 for s in t.stride()[:-1]) and t.data_ptr() % 16 == 0:
        return t
    return t.contiguous()


class _PrepFn(torch.autograd.Function):
    """Raw ``q, k, v, beta, g`` -> the scan operands ``W, U, QG, M, KD, GL`` (``[B*H, C, 64, ...]``)."""

    @staticmethod
    def forward(ctx, q, k, v, beta, g):
        q, k, v = _rows_ok(q), _rows_ok(k), _rows_ok(v)
        W, U, QG, M, KD, GL, T = ext().gdn_prep_fwd(q, k, v, beta, g)
        ctx.save_for_backward(q, k, v, beta, g, T)
        return W, U, QG, M, KD, GL

    @staticmethod
    def backward(ctx, dW, dU, dQG, dM, dKD, dGL):
        q, k, v, beta, g, T = ctx.saved_tensors
        grads = [t.contiguous() for t in (dW, dU, dQG, dM, dKD, dGL)]
        return tuple(ext().gdn_prep_bwd(q, k, v, beta, g, T, *grads))


def prep_torch(q, k, v, beta, g, chunk_size: int = _L):
    """The chunk-parallel stage as batched tensor algebra (one triangular solve for the WY inverse): the scan operands
    ``W, U, QG, M, KD, GL`` of :class:`_ScanFn`.  Fallback for shapes the kernel does not cover, and its test oracle."""
    B, H, S, dk = q.shape
    dv = v.shape[-1]
    L = chunk_size
    q = oracle.l2_normalize(q.float()) * dk ** -0.5
    k = oracle.l2_normalize(k.float())
    v, beta, g = v.float(), beta.float(), g.float()
    pad = (L - S % L) % L
    if pad:
        q, k, v = (TF.pad(t, (0, 0, 0, pad)) for t in (q, k, v))
        beta, g = TF.pad(beta, (0, pad)), TF.pad(g, (0, pad))
    C = q.shape[2] // L
    v_beta = (v * beta[..., None]).view(B, H, C, L, dv)
    k_beta = (k * beta[..., None]).view(B, H, C, L, dk)
    q, k = q.view(B, H, C, L, dk), k.view(B, H, C, L, dk)
    g = g.view(B, H, C, L).cumsum(-1)
    tril = torch.tril(torch.ones(L, L, device=q.device))
    decay = torch.exp((g[..., :, None] - g[..., None, :]).clamp(-30.0, 30.0)) * tril
    upper = torch.triu(torch.ones(L, L, dtype=torch.bool, device=q.device))
    attn = (-(k_beta @ k.transpose(-1, -2)) * decay).masked_fill(upper, 0.0)
    eye = torch.eye(L, device=q.device)
    # (I - attn)^-1: what the reference's row-by-row forward substitution computes, in one triangular solve
    T = torch.linalg.solve_triangular(eye - attn, eye.expand_as(attn).contiguous(), upper=False)
    g_exp = torch.exp(g.clamp(-30.0, 30.0))
    U = T @ v_beta
    W = T @ (k_beta * g_exp[..., None])
    k_decay = torch.exp((g[..., -1:] - g).clamp(-30.0, 30.0))
    strict_upper = torch.triu(torch.ones(L, L, dtype=torch.bool, device=q.device), diagonal=1)
    M = ((q @ k.transpose(-1, -2)) * decay).masked_fill(strict_upper, 0.0)
    QG = q * g_exp[..., None]
    KD = k * k_decay[..., None]
    GL = g_exp[..., -1]
    BH = B * H
    return (W.reshape(BH, C, L, dk), U.reshape(BH, C, L, dv), QG.reshape(BH, C, L, dk), M.reshape(BH, C, L, L),
            KD.reshape(BH, C, L, dk), GL.reshape(BH, C))


def chunk_gated_delta_rule_cuda(q, k, v, beta, g, chunk_size: int = _L) -> torch.Tensor:
    """q,k ``[B,H,S,dk]``, v ``[B,H,S,dv]``, beta,g ``[B,H,S]`` -> ``[B,H,S,dv]`` (fp32)."""
    B, H, S, dk = q.shape
    dv = v.shape[-1]
    L = chunk_size
    if prep_kernel_path(dk, dv):
        W, U, QG, M, KD, GL = _PrepFn.apply(q.float(), k.float(), v.float(), beta.float(), g.float())
        O = _ScanFn.apply(W, U, QG, M, KD, GL)
        return O.reshape(B, H, -1, dv)[:, :, :S]
    O = _ScanFn.apply(*prep_torch(q, k, v, beta, g, L))
    return O.reshape(B, H, -1, dv)[:, :, :S]
