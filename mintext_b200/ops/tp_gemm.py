"""Tensor-parallel projections whose collective runs inside the GEMM kernel (``csrc/comm/tp_gemm.cu``).

* ``ag_linear``: all-gather of the token shards folded into the first consuming GEMM.  Each rank publishes its
  shard in a symmetric buffer; after one in-kernel barrier the GEMM kernel's gather warps pull the peers' rows over
  NVLink with bulk TMA copies while its tensor-core warps start on the rows that are already local.  The gathered
  activations stay behind for the other projections of the same input and for the weight gradients.
* ``linear_rs``: the GEMM's epilogue stores each output tile directly into the staging slot of the rank that owns
  those token rows; after a barrier a local kernel adds the ``t`` slots.

Backward uses the same two kernels with the roles swapped (the data gradient of a column-parallel projection is
a GEMM + scatter, that of a row-parallel projection a gather + GEMM).  Symmetric buffers are double-buffered by call
parity, which makes one barrier per call sufficient: a rank reuses a buffer only two calls later, and every peer
has passed the barrier of the call in between after it finished reading.

The reference obtains these overlaps from XLA's collective-matmul and latency-hiding-scheduler flags
(mintext/utils/xla_flags.py:15-31); here they are explicit kernels.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from mintext_b200.ops._ext import ext, status_word

_ROW_BLOCK = 128


class TPWorkspace:
    def __init__(self, tp):
        import torch.distributed._symmetric_memory as symm

        self._symm = symm
        self.tp = tp
        self.group = tp.group
        self.rank, self.world = tp.rank, tp.size
        self.device = tp.device
        self.flags = symm.empty(64, dtype=torch.int32, device=self.device)
        self.flags.zero_()
        self._h_flags = symm.rendezvous(self.flags, self.group)
        self.flag_ptrs = [int(p) for p in self._h_flags.buffer_ptrs]
        self.seq = 0
        self._bufs: dict[str, tuple[torch.Tensor, list[int], object]] = {}
        self._ready: torch.Tensor | None = None
        self._ag_calls = 0
        self._rs_calls = 0
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)

    # ------------------------------------------------------------------ plumbing
    def barrier(self) -> None:
        self.seq += 1
        ext().symm_barrier(self.flag_ptrs, self.rank, self.seq, status_word(self.device))

    def _buffer(self, name: str, numel: int) -> tuple[torch.Tensor, list[int]]:
        """Symmetric bf16 buffer of at least ``numel`` elements.  Growing is collective: every rank runs the same
        sequence of calls with the same shapes, so all of them get here together."""
        cur = self._bufs.get(name)
        if cur is not None and cur[0].numel() >= numel:
            return cur[0], cur[1]
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)  # nobody still reads the buffer that is about to be replaced
        buf = self._symm.empty(numel, dtype=torch.bfloat16, device=self.device)
        handle = self._symm.rendezvous(buf, self.group)
        ptrs = [int(p) for p in handle.buffer_ptrs]
        self._bufs[name] = (buf, ptrs, handle)
        return buf, ptrs

    def _ready_counters(self, blocks: int) -> torch.Tensor:
        if self._ready is None or self._ready.numel() < blocks:
            self._ready = torch.zeros(max(blocks, 1024), dtype=torch.int32, device=self.device)
        return self._ready

    @staticmethod
    def supports(tokens_local: int, k: int, n: int) -> bool:
        return tokens_local % _ROW_BLOCK == 0 and k % 64 == 0 and n % 8 == 0

    # ------------------------------------------------------------------ fused ops
    def gather_gemm(self, x_local: torch.Tensor, w: torch.Tensor, b_kn: bool) -> tuple[torch.Tensor, torch.Tensor]:
        """``(gathered [T, K], gathered @ W)`` with ``W`` given as ``[K, N]`` (``b_kn``) or ``[N, K]``."""
        Tl, K = x_local.shape
        T = Tl * self.world
        N = w.shape[1] if b_kn else w.shape[0]
        parity = self._ag_calls & 1
        self._ag_calls += 1
        shard, ptrs = self._buffer(f"shard{parity}", Tl * K)
        shard[: Tl * K].view(Tl, K).copy_(x_local)
        ready = self._ready_counters(T // _ROW_BLOCK)
        ready.zero_()
        self.barrier()  # every rank's shard is in place
        xg = torch.empty(T, K, dtype=torch.bfloat16, device=self.device)
        y = torch.empty(T, N, dtype=torch.bfloat16, device=self.device)
        ext().tp_gemm_ag(ptrs, xg, w, y, b_kn, self.rank, ready, status_word(self.device))
        return xg, y

    def gemm_scatter(self, x: torch.Tensor, w: torch.Tensor, b_kn: bool) -> torch.Tensor:
        """Rows ``[r*T/t, (r+1)*T/t)`` of ``sum over ranks (x @ W)``."""
        T, _ = x.shape
        N = w.shape[1] if b_kn else w.shape[0]
        Tl = T // self.world
        parity = self._rs_calls & 1
        self._rs_calls += 1
        staging, ptrs = self._buffer(f"stage{parity}", self.world * Tl * N)
        slot_bytes = Tl * N * 2
        slot_ptrs = [p + self.rank * slot_bytes for p in ptrs]  # this rank's slot in every peer's staging buffer
        ext().tp_gemm_rs(x, w, slot_ptrs, b_kn, self.rank, status_word(self.device))
        self.barrier()  # all partial tiles have landed in this rank's slots
        y = torch.empty(Tl, N, dtype=torch.bfloat16, device=self.device)
        ext().tp_reduce_slots(staging[: self.world * Tl * N], y)
        return y


def _gemm(a, b, c, a_km, b_kn, accumulate=False):
    ext().gemm(a, b, c, a_km, b_kn, accumulate, status_word(a.device))
    return c


class _AGLinearFn(torch.autograd.Function):
    """``(gathered, gathered @ W_0, gathered @ W_1, ...)`` for column-parallel kernels ``W_i [K, N_i]``."""

    @staticmethod
    def forward(ctx, x_local, ws, n, *rest):
        weights, main_grads = rest[:n], rest[n:]
        xg, y0 = ws.gather_gemm(x_local, weights[0], True)
        outs = [y0]
        for w in weights[1:]:
            outs.append(_gemm(xg, w, torch.empty(xg.shape[0], w.shape[1], dtype=torch.bfloat16, device=xg.device),
                              False, True))
        ctx.ws, ctx.n, ctx.main_grads = ws, n, main_grads
        ctx.save_for_backward(xg, *weights)
        ctx.mark_non_differentiable(xg)
        ctx.set_materialize_grads(False)
        return (xg, *outs)

    @staticmethod
    def backward(ctx, _dxg, *dys):
        xg, *weights = ctx.saved_tensors
        live = [(dy.contiguous(), w, mg) for dy, w, mg in zip(dys, weights, ctx.main_grads) if dy is not None]
        dx = None
        if ctx.needs_input_grad[0] and live:
            if len(live) == 1:
                dy_cat, w_cat = live[0][0], live[0][1]
            else:
                dy_cat = torch.cat([d for d, _, _ in live], dim=1)
                w_cat = torch.cat([w for _, w, _ in live], dim=1)
            dx = ctx.ws.gemm_scatter(dy_cat, w_cat, False)  # dy [T, sumN] . W_cat [K, sumN]^T, scattered to owners
        dws = []
        for dy, w, mg in zip(dys, weights, ctx.main_grads):
            if dy is None:
                dws.append(None)
            elif mg is not None:
                _gemm(xg, dy.contiguous(), mg.view(w.shape), True, True, accumulate=True)
                dws.append(None)
            else:
                dw = torch.empty(w.shape, device=w.device, dtype=torch.float32)
                dws.append(_gemm(xg, dy.contiguous(), dw, True, True).to(w.dtype))
        return (dx, None, None, *dws, *([None] * ctx.n))


class _LinearRSFn(torch.autograd.Function):
    """Token shard of ``sum over ranks (x [T, K_local] @ W [K_local, N])``."""

    @staticmethod
    def forward(ctx, x, w, ws, main_grad):
        ctx.ws, ctx.main_grad = ws, main_grad
        ctx.save_for_backward(x, w)
        return ws.gemm_scatter(x, w, True)

    @staticmethod
    def backward(ctx, dy_local):
        x, w = ctx.saved_tensors
        dyg, dx = ctx.ws.gather_gemm(dy_local.contiguous(), w, False)  # gather(dy) [T, N] . W [K_local, N]^T
        dw = None
        if ctx.main_grad is not None:
            _gemm(x, dyg, ctx.main_grad.view(w.shape), True, True, accumulate=True)
        else:
            dw = torch.empty(w.shape, device=w.device, dtype=torch.float32)
            dw = _gemm(x, dyg, dw, True, True).to(w.dtype)
        return dx, dw, None, None


def ag_linear(x_local: torch.Tensor, weights: list[torch.Tensor], tp):
    """Returns ``(gathered, [gathered @ W for W in weights])``; ``weights`` are 2-D ``[K, N_i]`` (a ``main_grad``
    attribute on a weight receives its gradient)."""
    ws = tp.comm()
    x2 = x_local if x_local.is_contiguous() else x_local.contiguous()
    mgs = [getattr(w, "main_grad", None) for w in weights]
    out = _AGLinearFn.apply(x2, ws, len(weights), *weights, *mgs)
    return out[0], list(out[1:])


def linear_rs(x: torch.Tensor, weight: torch.Tensor, tp) -> torch.Tensor:
    ws = tp.comm()
    x2 = x if x.is_contiguous() else x.contiguous()
    return _LinearRSFn.apply(x2, weight, ws, getattr(weight, "main_grad", None))


# ---------------------------------------------------------------------------------------------- sharded weights
class ShardedWeight:
    """A ``[K, N]`` kernel stored 1/world per rank (rows ``[r*K/w, (r+1)*K/w)``) in symmetric memory, for fully
    sharded data parallelism without a resident full copy.  ``fsdp_linear`` gathers it inside the GEMM kernel:
    the gather warps pull the peers' rows over NVLink while the main loop starts on this rank's own k-blocks.

    The reference gets this overlap from XLA's async all-gather + latency-hiding scheduler
    (mintext/utils/xla_flags.py:15-31) on ``fsdp``-sharded kernels (mintext/distributed/sharding.py:33-47)."""

    def __init__(self, full: torch.Tensor, group, device):
        import torch.distributed._symmetric_memory as symm

        self.group = group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        K, N = full.shape
        if K % (64 * self.world) != 0 or N % 128 != 0:
            raise ValueError("ShardedWeight needs K % (64 * world) == 0 and N % 128 == 0")
        self.shape = (K, N)
        self.device = torch.device(device)
        rows = K // self.world
        self.shard = symm.empty((rows, N), dtype=torch.bfloat16, device=self.device)
        self.shard.copy_(full[self.rank * rows:(self.rank + 1) * rows].to(self.device, torch.bfloat16))
        self.shard.requires_grad_(True)
        self._handle = symm.rendezvous(self.shard, group)
        self.ptrs = [int(p) for p in self._handle.buffer_ptrs]
        self.ready = torch.zeros(K // 64, dtype=torch.int32, device=self.device)
        torch.cuda.synchronize(self.device)
        dist.barrier(group=group)  # every shard is in place; callers barrier again after they update shards


class _FsdpLinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, shard, sw):
        K, N = sw.shape
        w_full = torch.empty(K, N, dtype=torch.bfloat16, device=x.device)
        y = torch.empty(x.shape[0], N, dtype=torch.bfloat16, device=x.device)
        sw.ready.zero_()
        ext().fsdp_gemm_agw(x, sw.ptrs, w_full, y, sw.rank, sw.ready, status_word(x.device))
        ctx.save_for_backward(x, w_full)
        ctx.sw = sw
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w_full = ctx.saved_tensors
        sw = ctx.sw
        dy = dy.contiguous()
        dx = _gemm(dy, w_full, torch.empty_like(x), False, False)
        dw_full = _gemm(x, dy, torch.empty(sw.shape, dtype=torch.float32, device=x.device), True, True)
        dw = torch.empty(sw.shape[0] // sw.world, sw.shape[1], dtype=torch.float32, device=x.device)
        dist.reduce_scatter_tensor(dw, dw_full, group=sw.group)
        return dx, dw.to(torch.bfloat16), None


def fsdp_linear(x: torch.Tensor, sw: ShardedWeight) -> torch.Tensor:
    """``x [T, K] @ W [K, N]`` with ``W`` all-gathered from its row shards inside the GEMM kernel."""
    x2 = x if x.is_contiguous() else x.contiguous()
    return _FsdpLinearFn.apply(x2, sw.shard, sw)
