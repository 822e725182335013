"""CUDA front-ends of the MoE ops (permute, grouped GEMM, transposed grouped GEMM).

``cuda_path`` gates them: until a tensor is CUDA bf16 (and the backend is not forced to the oracle) the callers
in :mod:`mintext_b200.kernels` use the plain-PyTorch statements instead.
"""

from __future__ import annotations

import torch

from . import functional as F
from . import oracle
from ._ext import ext, status_word


def cuda_path(x: torch.Tensor) -> bool:
    return x.is_cuda and x.dtype == torch.bfloat16 and F._backend() != "oracle" and hasattr(ext(), "grouped_gemm")


def _offsets(group_sizes: torch.Tensor) -> torch.Tensor:
    off = torch.zeros(group_sizes.numel() + 1, dtype=torch.int32, device=group_sizes.device)
    off[1:] = torch.cumsum(group_sizes, 0)
    return off


class _GroupedFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, group_sizes, main_grad):
        off = _offsets(group_sizes)
        y = torch.empty(x.shape[0], w.shape[2], device=x.device, dtype=torch.bfloat16)
        ext().grouped_gemm(x, w, y, off, True, status_word(x.device))
        ctx.save_for_backward(x, w, off)
        ctx.main_grad = main_grad
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, off = ctx.saved_tensors
        dy = dy.contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = torch.empty_like(x)
            # dy[M,N] . w[e][K,N]^T : w[e] rows are K-major for this product
            ext().grouped_gemm(dy, w, dx, off, False, status_word(x.device))
        if ctx.needs_input_grad[1]:
            mg = ctx.main_grad
            if mg is not None:
                ext().grouped_wgrad(x, dy, mg.view(w.shape), off, True, status_word(x.device))
            else:
                dwf = torch.zeros(w.shape, device=w.device, dtype=torch.float32)
                ext().grouped_wgrad(x, dy, dwf, off, False, status_word(x.device))
                dw = dwf.to(w.dtype)
        return dx, dw, None, None


def grouped_matmul_cuda(x, w, group_sizes):
    return _GroupedFn.apply(x.contiguous(), w, group_sizes, getattr(w, "main_grad", None))


def tgmm_cuda(lhs, rhs, group_sizes):
    out = torch.zeros(group_sizes.numel(), lhs.shape[1], rhs.shape[1], device=lhs.device, dtype=torch.float32)
    ext().grouped_wgrad(lhs.contiguous(), rhs.contiguous(), out, _offsets(group_sizes), False, status_word(lhs.device))
    return out.to(lhs.dtype)


class _RouteFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, tokens, topk_idx, num_experts):
        N, K = topk_idx.shape
        flat = topk_idx.reshape(-1)
        sort_idx = torch.argsort(flat, stable=True)
        sizes = torch.bincount(flat, minlength=num_experts)
        src_token = torch.div(sort_idx, K, rounding_mode="floor")
        rows = tokens.index_select(0, src_token)
        ctx.save_for_backward(sort_idx)
        ctx.meta = (N, K)
        ctx.mark_non_differentiable(sort_idx, sizes)
        return rows, sort_idx, sizes

    @staticmethod
    def backward(ctx, drows, _a, _b):
        (sort_idx,) = ctx.saved_tensors
        N, K = ctx.meta
        inv = torch.empty_like(sort_idx)
        inv[sort_idx] = torch.arange(sort_idx.numel(), device=sort_idx.device)
        return drows.index_select(0, inv).view(N, K, -1).sum(1), None, None


def route_cuda(tokens, topk_idx, num_experts):
    return _RouteFn.apply(tokens, topk_idx, num_experts)


def unroute_cuda(sorted_out, sort_idx, topk_w, K):
    return oracle.unroute(sorted_out, sort_idx, topk_w, K)
