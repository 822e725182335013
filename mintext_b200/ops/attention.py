"""Flash-attention front-end: autograd wrapper around the tcgen05 forward / backward kernels."""

from __future__ import annotations

import torch

from ._ext import ext, status_word


def flash_supported(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> bool:
    """Forward and backward kernels cover head dims 64, 128 and 256 and the multi-head-latent shape (192-wide queries
    and keys, 128-wide values): the kernel path takes bf16 tensors of those shapes with sequence lengths that are
    multiples of 128, anything else goes to the oracle."""
    if not hasattr(ext(), "flash_fwd"):
        return False
    d, dv = q.shape[-1], v.shape[-1]
    return (q.dtype == torch.bfloat16 and (d, dv) in ((64, 64), (128, 128), (256, 256), (192, 128)) and k.shape[-1] == d
            and q.shape[1] % 128 == 0 and k.shape[1] == q.shape[1] and q.shape[2] % k.shape[2] == 0)


class _FlashFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, scale, causal, window, softcap):
        B, S, H, d = q.shape
        o = torch.empty(B, S, H, v.shape[-1], device=q.device, dtype=torch.bfloat16)
        lse = torch.empty(B, H, S, device=q.device, dtype=torch.float32)
        ext().flash_fwd(q, k, v, o, lse, float(scale), bool(causal), int(window or 0), float(softcap or 0.0),
                        status_word(q.device))
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.meta = (float(scale), bool(causal), int(window or 0), float(softcap or 0.0))
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse = ctx.saved_tensors
        scale, causal, window, softcap = ctx.meta
        do = do.contiguous()
        B, S, H, d = q.shape
        dq = torch.empty(B, S, H, d, device=q.device, dtype=q.dtype)
        dk = torch.empty(B, S, k.shape[2], d, device=q.device, dtype=q.dtype)
        dv = torch.empty(B, S, k.shape[2], v.shape[-1], device=q.device, dtype=q.dtype)
        dq_accum = torch.empty(B * S, H, d, device=q.device, dtype=torch.float32)  # cleared by the pre-pass
        delta = torch.empty_like(lse)
        ext().flash_bwd(q, k, v, o, lse, do, dq, dk, dv, dq_accum, delta, scale, causal, window, softcap,
                        status_word(q.device))
        return dq, dk, dv, None, None, None, None


def _packed(t: torch.Tensor) -> torch.Tensor:
    """The kernels take any token pitch but want the heads of a token back to back."""
    ok = (t.stride(3) == 1 and t.stride(2) == t.shape[3] and t.stride(0) == t.stride(1) * t.shape[1]
          and t.stride(1) % 8 == 0 and t.data_ptr() % 16 == 0)
    return t if ok else t.contiguous()


def flash_attention(q, k, v, scale, causal=True, window=None, softcap=None):
    """q ``[B,S,H,d]``, k/v ``[B,S,Hkv,d]`` (any row pitch, unit inner stride) -> ``[B,S,H,d]``."""
    q, k, v = _packed(q), _packed(k), _packed(v)
    return _FlashFn.apply(q, k, v, scale, causal, window, softcap)
