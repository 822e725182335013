"""Ragged grouped matmul and its transposed (weight-gradient) form
(reference: mintext/kernels/grouped_matmul.py).

* ``grouped_matmul(x[M,Kin], w[E,Kin,Kout], group_sizes[E]) -> [M,Kout]``
* ``grouped_matmul_vjp``: same product with an explicit backward: dlhs is a grouped matmul against ``w^T``,
  drhs is ``tgmm`` (a true per-expert reduction over the ragged row segment, not the reference's dense
  one-hot einsum that costs E times the FLOPs).
* ``tgmm(lhs[M,K], rhs[M,N], group_sizes[E]) -> [E,K,N]``

``tiling = (tile_m, tile_k, tile_n)`` selects between the two tilings the tcgen05 grouped kernel exists in:
``(128, 64, 256)`` single-CTA tiles, ``(256, 64, 256)`` CTA-pair tiles on two SMs (``cta_group::2``); other values,
or None, keep the default.  On CPU the argument has no effect.
"""

from __future__ import annotations

import torch

from mintext_b200.ops import oracle


def _cuda(x: torch.Tensor) -> bool:
    from mintext_b200.ops import moe as moe_ops

    return moe_ops.cuda_path(x)


def grouped_matmul(x: torch.Tensor, weights: torch.Tensor, group_sizes: torch.Tensor, *, tiling=None) -> torch.Tensor:
    return grouped_matmul_vjp(x, weights, group_sizes, tiling=tiling)


def tgmm(lhs: torch.Tensor, rhs: torch.Tensor, group_sizes: torch.Tensor, *, tiling=None) -> torch.Tensor:
    if _cuda(lhs):
        from mintext_b200.ops import moe as moe_ops

        return moe_ops.tgmm_cuda(lhs, rhs, group_sizes)
    return oracle.tgmm(lhs, rhs, group_sizes)


class _GroupedMatmulFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, group_sizes):
        ctx.save_for_backward(x, w, group_sizes)
        return oracle.grouped_matmul(x, w, group_sizes)

    @staticmethod
    def backward(ctx, dy):
        x, w, group_sizes = ctx.saved_tensors
        dx = oracle.grouped_matmul(dy, w.transpose(1, 2), group_sizes) if ctx.needs_input_grad[0] else None
        dw = oracle.tgmm(x, dy, group_sizes).to(w.dtype) if ctx.needs_input_grad[1] else None
        return dx, dw, None


def grouped_matmul_vjp(x: torch.Tensor, weights: torch.Tensor, group_sizes: torch.Tensor, *, tiling=None,
                       mosaic_fusion: bool = True) -> torch.Tensor:
    if _cuda(x):
        from mintext_b200.ops import moe as moe_ops

        return moe_ops.grouped_matmul_cuda(x, weights, group_sizes, tiling)
    return _GroupedMatmulFn.apply(x, weights.to(x.dtype), group_sizes)
