"""Tensor parallelism with token-sharded activations (Megatron-style TP + sequence parallelism).

Inside a tensor-parallel group of ``t`` ranks the residual stream is sharded over tokens: a rank holds rows
``[r*T/t, (r+1)*T/t)`` of the flattened ``[T, D]`` activations of the group's batch.  A layer's column-parallel
projections (query/key/value heads, MLP gate/up columns) consume the *gathered* tokens and produce this rank's
slice of the features; its row-parallel projections (attention output, MLP down) produce partial sums over all
tokens that are reduce-scattered back to the token shards:

    x_local --norm--> all-gather --> [q|k|v]_local heads --> attention --> out_local --> reduce-scatter --> + x_local

Embedding, norms and the output head are replicated and operate on the local tokens only, so the tensor-parallel
ranks behave like data-parallel ranks for them (their gradients are reduced over every rank of the job).

``all_gather_tokens`` / ``reduce_scatter_tokens`` are differentiable (each is the other's backward).  On CUDA with
``fused=True`` the projections call the fused kernels in :mod:`mintext_b200.ops.tp_gemm` (all-gather folded into
the consuming GEMM, GEMM epilogue scattering partial tiles to their owners); otherwise NCCL / gloo collectives
around ordinary GEMMs, which is the baseline composition and the oracle.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

_CURRENT = None


def current_tp():
    return _CURRENT


def set_current_tp(ctx) -> None:
    global _CURRENT
    _CURRENT = ctx


class TensorParallel:
    def __init__(self, group, device, fused: bool = True):
        self.group = group
        self.size = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.device = torch.device(device)
        self.fused = bool(fused) and self.device.type == "cuda" and self.size <= 8
        self._comm = None

    def shard(self, n: int, what: str) -> tuple[int, int]:
        if n % self.size != 0:
            raise ValueError(f"{what} ({n}) must be divisible by the tensor-parallel size ({self.size})")
        per = n // self.size
        return self.rank * per, (self.rank + 1) * per

    def comm(self):
        """Peer-memory workspace of the fused kernels (created on first use)."""
        if self._comm is None:
            from mintext_b200.ops.tp_gemm import TPWorkspace

            self._comm = TPWorkspace(self)
        return self._comm


class _AllGatherTokens(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        n = dist.get_world_size(group)
        out = torch.empty((n * x.shape[0],) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out, x.contiguous(), group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        return _reduce_scatter(g.contiguous(), ctx.group), None


class _GatherForReplicated(torch.autograd.Function):
    """All-gather of the token shards in front of a sub-layer that every rank of the group computes in full (it has
    no sharded kernel path).  The full computation back-propagates the gradient of the *sum* of the ranks' losses,
    the same on every rank, so the backward is just this rank's rows - no reduction."""

    @staticmethod
    def forward(ctx, x, tp):
        ctx.tp = tp
        out = torch.empty((tp.size * x.shape[0],) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out, x.contiguous(), group=tp.group)
        return out

    @staticmethod
    def backward(ctx, g):
        n = g.shape[0] // ctx.tp.size
        return g[ctx.tp.rank * n:(ctx.tp.rank + 1) * n].contiguous(), None


class _SliceFromReplicated(torch.autograd.Function):
    """This rank's token rows of a replicated sub-layer's output; backward gathers every rank's output gradient so
    that the replicated backward sees all of them."""

    @staticmethod
    def forward(ctx, y, tp):
        ctx.tp = tp
        n = y.shape[0] // tp.size
        return y[tp.rank * n:(tp.rank + 1) * n].contiguous()

    @staticmethod
    def backward(ctx, g):
        tp = ctx.tp
        out = torch.empty((tp.size * g.shape[0],) + tuple(g.shape[1:]), dtype=g.dtype, device=g.device)
        dist.all_gather_into_tensor(out, g.contiguous(), group=tp.group)
        return out, None


def run_replicated(fn, h: torch.Tensor, tp: "TensorParallel"):
    """Run ``fn`` (a sub-layer without a tensor-parallel kernel path: multi-head-latent attention, Gated Delta Rule,
    mixture of experts) on the whole ``[B, S, D]`` batch on every rank of the group and return this rank's token
    rows of its output (plus ``fn``'s auxiliary output, if it returns a pair).  The parameters of such a sub-layer
    carry ``tp_replicated_compute``: their gradients are identical on all ranks of the group and the engine divides
    them by the group size before the cross-rank sum."""
    B, S = tp.batch_shape
    D = h.shape[-1]
    full = _GatherForReplicated.apply(h.reshape(-1, D), tp).view(B, S, D)
    out = fn(full)
    aux = None
    if isinstance(out, tuple):
        out, aux = out
    return _SliceFromReplicated.apply(out.reshape(B * S, -1), tp).view(1, -1, out.shape[-1]), aux


def mark_replicated(module: torch.nn.Module) -> None:
    for p in module.parameters():
        p.tp_replicated_compute = True


class _ReduceScatterTokens(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return _reduce_scatter(x.contiguous(), group)

    @staticmethod
    def backward(ctx, g):
        n = dist.get_world_size(ctx.group)
        out = torch.empty((n * g.shape[0],) + tuple(g.shape[1:]), dtype=g.dtype, device=g.device)
        dist.all_gather_into_tensor(out, g.contiguous(), group=ctx.group)
        return out, None


def _reduce_scatter(x: torch.Tensor, group) -> torch.Tensor:
    n, r = dist.get_world_size(group), dist.get_rank(group)
    per = x.shape[0] // n
    if x.is_cuda:
        out = torch.empty((per,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.reduce_scatter_tensor(out, x, group=group)
        return out
    y = x.clone()  # gloo has no reduce-scatter
    dist.all_reduce(y, group=group)
    return y[r * per:(r + 1) * per].clone()


def all_gather_tokens(x: torch.Tensor, tp: TensorParallel) -> torch.Tensor:
    """``[T/t, ...] -> [T, ...]`` (rows of rank 0 first)."""
    return _AllGatherTokens.apply(x, tp.group)


def reduce_scatter_tokens(x: torch.Tensor, tp: TensorParallel) -> torch.Tensor:
    """``[T, ...]`` partial sums on every rank ``-> [T/t, ...]`` complete sums of this rank's rows."""
    return _ReduceScatterTokens.apply(x, tp.group)


def as_matrix(kernel: torch.Tensor, rows: int) -> torch.Tensor:
    """2-D ``[rows, -1]`` view of a (possibly head-shaped) kernel that keeps the engine's ``main_grad`` attribute."""
    if kernel.dim() == 2 and kernel.shape[0] == rows:
        return kernel
    w2 = kernel.reshape(rows, -1)
    if hasattr(kernel, "main_grad"):
        w2.main_grad = kernel.main_grad
    return w2


def _fusable(tp: TensorParallel, x: torch.Tensor, weights, tokens_local: int, k: int) -> bool:
    from mintext_b200.ops import functional as F

    return (tp.fused and F.use_cuda(x) and x.dtype == torch.bfloat16 and tokens_local % 128 == 0 and k % 64 == 0
            and all(w.dtype == torch.bfloat16 and w.shape[0] % 8 == 0 and w.shape[1] % 8 == 0 for w in weights))


def column_linear(x_local: torch.Tensor, weights: list[torch.Tensor], tp: TensorParallel, dtype, names=None):
    """Gather the token shards once and apply several column-parallel kernels ``[D, out_local...]`` to them.
    Returns the gathered input (kept for the weight gradients) and one output per kernel."""
    from mintext_b200.ops import functional as F

    if _fusable(tp, x_local, weights, x_local.shape[0], x_local.shape[1]):
        from mintext_b200.ops import tp_gemm

        return tp_gemm.ag_linear(x_local, weights, tp)
    xg = all_gather_tokens(x_local, tp)
    names = names or [None] * len(weights)
    return xg, [F.linear(xg, w, name=n, dtype=dtype) for w, n in zip(weights, names)]


def row_linear(x: torch.Tensor, weight: torch.Tensor, tp: TensorParallel, dtype, name=None) -> torch.Tensor:
    """Row-parallel projection: ``x [T, in_local] @ W [in_local, D]`` summed over ranks, scattered to token shards."""
    from mintext_b200.ops import functional as F

    if _fusable(tp, x, [weight], x.shape[0] // tp.size, weight.shape[1]):
        from mintext_b200.ops import tp_gemm

        return tp_gemm.linear_rs(x, weight, tp)
    return reduce_scatter_tokens(F.linear(x, weight, name=name, dtype=dtype), tp)
