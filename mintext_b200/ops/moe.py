"""CUDA path of the MoE ops: padded expert-contiguous dispatch, tcgen05 grouped GEMMs, weighted combine.

The grouped kernels want every expert's rows to start at a multiple of 128, so dispatch writes the ``N*K``
(token, slot) rows into a buffer where each expert's group is padded with zero rows.  All index arithmetic
(stable order inside an expert, padded offsets, destinations) stays on the device: the buffer is sized for the
worst case ``N*K + E*127`` rows, so nothing has to be read back to the host.
"""

from __future__ import annotations

import torch

from . import functional as F
from . import oracle
from ._ext import ext, status_word

_PAD = 128


def cuda_path(x: torch.Tensor) -> bool:
    return x.is_cuda and x.dtype == torch.bfloat16 and F._backend() != "oracle" and hasattr(ext(), "grouped_gemm")


def _cumsum0(v: torch.Tensor) -> torch.Tensor:
    out = torch.zeros(v.numel() + 1, dtype=torch.int64, device=v.device)
    out[1:] = torch.cumsum(v, 0)
    return out


def padded_offsets(group_sizes: torch.Tensor):
    """``(int32 padded offsets [E+1], int64 unpadded offsets [E+1])``."""
    padded = (group_sizes + (_PAD - 1)) // _PAD * _PAD
    return _cumsum0(padded).to(torch.int32), _cumsum0(group_sizes)


def capacity(rows: int, num_experts: int) -> int:
    return (rows + num_experts * (_PAD - 1) + _PAD - 1) // _PAD * _PAD


def row_destinations(sorted_experts: torch.Tensor, off_p: torch.Tensor, off_u: torch.Tensor) -> torch.Tensor:
    """Position in the padded buffer of every row of the expert-sorted (unpadded) order."""
    r = torch.arange(sorted_experts.numel(), device=sorted_experts.device)
    return off_p.long()[sorted_experts] + (r - off_u[sorted_experts])


def tiling_variant(tiling) -> int:
    """Kernel variant a ``(tile_m, tile_k, tile_n)`` triple selects: tile_m 128 = the single-CTA grouped kernel
    (128 x 256 x 64 tiles), 256 = the CTA-pair kernel (256 x 256 x 64 on two SMs); anything else (or None) leaves
    the default choice.  These are the two tilings the tcgen05 grouped GEMM exists in, and what the autotuner picks
    between per projection."""
    if not tiling:
        return 0
    return {128: 1, 256: 2}.get(int(tiling[0]), 0)


class _variant:
    """Selects the grouped-kernel variant for the launches issued inside the block (per calling thread)."""

    def __init__(self, v: int):
        self.v = int(v)

    def __enter__(self):
        if self.v:
            ext().set_grouped_variant(self.v)

    def __exit__(self, *exc):
        if self.v:
            ext().set_grouped_variant(0)


class _GroupedPaddedFn(torch.autograd.Function):
    """``y = x @ w[e]`` on a padded, expert-contiguous row buffer (forward, data gradient and weight gradient all
    run the tcgen05 grouped kernel)."""

    @staticmethod
    def forward(ctx, x, w, off_p, main_grad, variant=0):
        y = torch.empty(x.shape[0], w.shape[2], device=x.device, dtype=torch.bfloat16)
        with _variant(variant):
            ext().grouped_gemm(x, w, y, off_p, True, status_word(x.device))
        ctx.save_for_backward(x, w, off_p)
        ctx.main_grad = main_grad
        ctx.variant = variant
        return y

    @staticmethod
    def backward(ctx, dy):
        with _variant(ctx.variant):
            return _GroupedPaddedFn._backward(ctx, dy) + (None,)

    @staticmethod
    def _backward(ctx, dy):
        x, w, off_p = ctx.saved_tensors
        dy = dy.contiguous()
        st = status_word(x.device)
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = torch.empty_like(x)
            ext().grouped_gemm(dy, w, dx, off_p, False, st)  # rows of w[e] ([K, N]) are K-major for dy @ w[e]^T
        if ctx.needs_input_grad[1]:
            mg = ctx.main_grad
            if mg is not None:
                ext().grouped_wgrad(x, dy, mg.view(w.shape), off_p, True, st)
            else:
                dwf = torch.zeros(w.shape, device=w.device, dtype=torch.float32)
                ext().grouped_wgrad(x, dy, dwf, off_p, False, st)
                dw = dwf.to(w.dtype)
        return dx, dw, None, None


class _GroupedMxfp8Fn(torch.autograd.Function):
    """``y = x @ w[e]`` on the padded expert layout with MXFP8 operands (e4m3 elements, one power-of-two scale per
    32 elements along the contraction, applied inside the tensor core: csrc/gemm/mxfp8_gemm.cu, grouped kernel).
    Forward and data gradient run in 8 bits - each operand quantised along the dimension its product contracts, the
    expert weights per expert with their own scale tiling; the weight gradient stays a bf16 grouped GEMM accumulating
    in fp32, as on the dense FP8 paths (mintext/modules/linear.py:37-57 for the layer semantics)."""

    @staticmethod
    def forward(ctx, x, w, off_p, main_grad):
        e, st = ext(), status_word(x.device)
        xq, xs, _, _ = e.mxfp8_quantize(x, True, False, False, False)
        # w [E, K, N]: the forward contracts K (transposed copy [E, N, K]), the data gradient contracts N (w as stored)
        wq, ws, wqt, wst = e.mxfp8_quantize_stack(w, True, True)
        ctx.save_for_backward(x, w, wq, ws, off_p)
        ctx.main_grad = main_grad
        return e.grouped_gemm_mxfp8(xq, xs, wqt, wst, off_p, st)

    @staticmethod
    def backward(ctx, dy):
        x, w, wq, ws, off_p = ctx.saved_tensors
        e, st = ext(), status_word(x.device)
        dy = dy.contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dyq, dys, _, _ = e.mxfp8_quantize(dy, True, False, False, False)
            dx = e.grouped_gemm_mxfp8(dyq, dys, wq, ws, off_p, st)   # dy [rows, N] . w[e] [K, N]^T
        if ctx.needs_input_grad[1]:
            mg = ctx.main_grad
            if mg is not None:
                e.grouped_wgrad(x, dy, mg.view(w.shape), off_p, True, st)
            else:
                dwf = torch.zeros(w.shape, device=w.device, dtype=torch.float32)
                e.grouped_wgrad(x, dy, dwf, off_p, False, st)
                dw = dwf.to(w.dtype)
        return dx, dw, None, None


def mxfp8_grouped_path(x_p: torch.Tensor, w: torch.Tensor) -> bool:
    """Shapes the block-scaled grouped kernel covers: both contraction lengths (forward K, data gradient N) in
    whole 128-element blocks."""
    return (x_p.is_cuda and x_p.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.dim() == 3
            and hasattr(ext(), "grouped_gemm_mxfp8") and w.shape[1] % 128 == 0 and w.shape[2] % 128 == 0
            and x_p.shape[0] % 128 == 0 and x_p.shape[0] // 128 <= 4096)


def grouped_padded(x_p: torch.Tensor, w: torch.Tensor, off_p: torch.Tensor, tiling=None, fp8: bool = False) -> torch.Tensor:
    if fp8 and mxfp8_grouped_path(x_p, w):
        return _GroupedMxfp8Fn.apply(x_p, w, off_p, getattr(w, "main_grad", None))
    return _GroupedPaddedFn.apply(x_p, w, off_p, getattr(w, "main_grad", None), tiling_variant(tiling))


def _pad_rows(x: torch.Tensor, group_sizes: torch.Tensor):
    E = group_sizes.numel()
    off_p, off_u = padded_offsets(group_sizes)
    experts = torch.repeat_interleave(torch.arange(E, device=x.device), group_sizes, output_size=x.shape[0])
    dest = row_destinations(experts, off_p, off_u)
    cap = capacity(x.shape[0], E)
    x_p = torch.zeros(cap, x.shape[1], device=x.device, dtype=x.dtype).index_copy(0, dest, x)
    return x_p, off_p, dest


def grouped_matmul_cuda(x, w, group_sizes, tiling=None):
    """Public ragged form: rows grouped by expert without padding."""
    x_p, off_p, dest = _pad_rows(x.contiguous(), group_sizes)
    return grouped_padded(x_p, w, off_p, tiling).index_select(0, dest)


def tgmm_cuda(lhs, rhs, group_sizes):
    l_p, off_p, _ = _pad_rows(lhs.contiguous(), group_sizes)
    r_p, _, _ = _pad_rows(rhs.contiguous(), group_sizes)
    out = torch.zeros(group_sizes.numel(), lhs.shape[1], rhs.shape[1], device=lhs.device, dtype=torch.float32)
    ext().grouped_wgrad(l_p, r_p, out, off_p, False, status_word(lhs.device))
    return out.to(lhs.dtype)


def route_cuda(tokens, topk_idx, num_experts):
    """Reference-shaped ``route`` (unpadded result) for API parity."""
    N, K = topk_idx.shape
    flat = topk_idx.reshape(-1)
    sort_idx = torch.argsort(flat, stable=True)
    sizes = torch.bincount(flat, minlength=num_experts)
    rows = tokens.index_select(0, torch.div(sort_idx, K, rounding_mode="floor"))
    return rows, sort_idx, sizes


def unroute_cuda(sorted_out, sort_idx, topk_w, K):
    return oracle.unroute(sorted_out, sort_idx, topk_w, K)


class _RouterFn(torch.autograd.Function):
    """Router kernels (``csrc/moe/route.cu``): ``kind`` 0 = sigmoid scores with group-limited top-k and selection
    bias (mintext/modules/moe.py:52-103), 1 = softmax top-k.  Returns ``(indices, weights fp32, scores fp32)``."""

    @staticmethod
    def forward(ctx, logits, bias, kind, top_k, n_group, topk_group, norm, scaling):
        idx, w, scores = ext().moe_router(logits, bias, kind, top_k, n_group, topk_group, norm, scaling)
        ctx.save_for_backward(scores, idx)
        ctx.meta = (kind, norm, scaling, logits.dtype)
        ctx.mark_non_differentiable(idx)
        ctx.set_materialize_grads(False)
        return idx, w, scores

    @staticmethod
    def backward(ctx, _didx, dw, dscores):
        scores, idx = ctx.saved_tensors
        kind, norm, scaling, dtype = ctx.meta
        if dw is None and dscores is None:
            return (None,) * 8
        dw = None if dw is None else dw.float().contiguous()
        dscores = None if dscores is None else dscores.float().contiguous()
        dlogits = ext().moe_router_bwd(scores, idx, dw, dscores, kind, norm, scaling)
        return dlogits.to(dtype), None, None, None, None, None, None, None


def router_cuda_path(logits: torch.Tensor, num_experts: int, top_k: int, n_group: int) -> bool:
    return (logits.is_cuda and logits.dtype in (torch.bfloat16, torch.float32) and F._backend() != "oracle"
            and hasattr(ext(), "moe_router") and num_experts <= 512 and top_k <= 16 and n_group <= 32)


def router_sigmoid_group(logits, bias, top_k, n_group, topk_group, norm_topk_prob, scaling):
    return _RouterFn.apply(logits.contiguous(), bias.float(), 0, int(top_k), int(n_group), int(topk_group),
                           bool(norm_topk_prob), float(scaling))


def router_softmax_topk(logits, top_k, norm_topk_prob, scaling: float = 1.0):
    """``(indices, weights, probs, aux)``; the Switch-style auxiliary loss ``E * sum_e f_e P_e`` is formed from the
    kernel's outputs (a histogram and a column mean)."""
    idx, w, probs = _RouterFn.apply(logits.contiguous(), None, 1, int(top_k), 0, 0, bool(norm_topk_prob), float(scaling))
    N, E = probs.shape
    f = oracle.histogram(idx, E).float() / (N * top_k)
    aux = E * (f * probs.mean(0)).sum()
    return idx, w, probs, aux


class _DispatchFn(torch.autograd.Function):
    """Token rows into the padded expert-contiguous layout; backward sums the K row gradients of a token."""

    @staticmethod
    def forward(ctx, x, src, pos, K):
        ctx.save_for_backward(pos)
        ctx.meta = (x.shape[0], K)
        return ext().moe_gather_rows(x, src, None, K)

    @staticmethod
    def backward(ctx, drows):
        (pos,) = ctx.saved_tensors
        N, K = ctx.meta
        dx, _ = ext().moe_combine_rows(drows.contiguous(), pos, None, N, K, True, None)
        return dx, None, None, None


class _CombineFn(torch.autograd.Function):
    """``out[n] = sum_k w[n,k] * y[pos[n,k]]``; backward scatters ``w * dout`` back to the padded rows and forms
    ``dw[n,k] = <y[pos[n,k]], dout[n]>``."""

    @staticmethod
    def forward(ctx, y, w, pos, src, K):
        N = w.shape[0]
        w32 = w.float().contiguous()
        ctx.save_for_backward(y, w32, pos, src)
        ctx.meta = (N, K, w.dtype)
        out, _ = ext().moe_combine_rows(y, pos, w32, N, K, True, None)
        return out

    @staticmethod
    def backward(ctx, dout):
        y, w32, pos, src = ctx.saved_tensors
        N, K, wdt = ctx.meta
        dout = dout.contiguous()
        dy = dw = None
        if ctx.needs_input_grad[0]:
            dy = ext().moe_gather_rows(dout, src, w32.reshape(-1), K)
        if ctx.needs_input_grad[1]:
            _, dw = ext().moe_combine_rows(y, pos, None, N, K, False, dout)
            dw = dw.to(wdt)
        return dy, dw, None, None, None


def sort_by_expert(topk_idx: torch.Tensor, num_experts: int):
    """Stable counting sort of the ``N*K`` (token, slot) entries by expert, on the device.  Returns
    ``(sizes int64 [E], padded offsets int32 [E+1], pos int64 [N*K], src int32 [capacity])`` where ``pos`` is the
    padded row of every entry and ``src`` the entry held by every padded row (-1 for padding)."""
    flat = topk_idx.reshape(-1).contiguous()
    cap = capacity(flat.numel(), num_experts)
    return ext().moe_sort(flat, num_experts, cap)


def experts_forward(x: torch.Tensor, topk_idx: torch.Tensor, topk_w: torch.Tensor, gate_up: torch.Tensor,
                    down: torch.Tensor, act: str, gate_up_tiling=None, down_tiling=None, fp8: bool = False) -> torch.Tensor:
    """Routed-expert MLP for ``x [N, D]``: counting-sort dispatch into the padded layout, two grouped GEMMs around
    the gated activation, weighted combine back to token order.  Differentiable end to end; every step is a kernel
    of this package."""
    N, K = topk_idx.shape
    E = gate_up.shape[0]
    sizes, off_p, pos, src = sort_by_expert(topk_idx, E)
    rows = _DispatchFn.apply(x.contiguous(), src, pos, K)
    h = grouped_padded(rows, gate_up, off_p, gate_up_tiling, fp8)
    h = F.gated_act(h, act)
    y = grouped_padded(h, down, off_p, down_tiling, fp8)
    return _CombineFn.apply(y, topk_w, pos, src, K)
