"""Expert parallelism: experts are distributed over the ranks of an ``expert`` group, tokens travel to them.

Two exchange implementations with identical results:

* **peer-memory path** (CUDA, symmetric memory): a rank computes, entirely on the device, where each of its
  ``N*K`` (token, slot) rows belongs in the *destination* rank's expert-contiguous, 128-padded input buffer and
  stores the row there with ``ep_push_rows``; the routing permute and the all-to-all are one pass, there is no
  host synchronisation and no regrouping on the receiver.  After the grouped GEMMs the expert outputs stay in
  place and the token's home rank pulls its K rows (``ep_pull_rows``) and reduces them with the routing weights.
  The backward pass mirrors this (push of output gradients, pull of input gradients).  Buffers hold
  ``capacity_factor * N*K`` rows; a destination that would overflow is reported through a status flag, never
  written out of bounds.
* **collective path** (any backend, also gloo on CPU): all-gather of tokens and routing, every rank serves the
  slots that chose its experts, reduce-scatter of the partial outputs.  This is the baseline composition and the
  oracle for the peer-memory path.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

_CURRENT = None


def current_ep():
    """The process-wide expert-parallel context, or None (single-rank experts)."""
    return _CURRENT


def set_current_ep(ctx) -> None:
    global _CURRENT
    _CURRENT = ctx


class ExpertParallel:
    def __init__(self, group, device: torch.device, capacity_factor: float = 2.0, fused: bool = True):
        self.group = group
        self.size = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.device = torch.device(device)
        self.capacity_factor = capacity_factor
        self.fused = bool(fused) and self.device.type == "cuda" and self.size <= 8
        self._bufs = None  # (cap_rows, dim) -> symmetric buffers
        self.seq = 0
        self.overflow = None
        self._dropped = None

    def local_expert_range(self, num_experts: int) -> tuple[int, int]:
        if num_experts % self.size != 0:
            raise ValueError(f"num_experts ({num_experts}) must be divisible by the expert-parallel size ({self.size})")
        per = num_experts // self.size
        return self.rank * per, (self.rank + 1) * per

    # ------------------------------------------------------------------ symmetric buffers
    def buffers(self, cap_rows: int, dim: int):
        if self._bufs is not None and self._bufs["cap"] >= cap_rows and self._bufs["dim"] == dim:
            return self._bufs
        import torch.distributed._symmetric_memory as symm

        from mintext_b200.ops._ext import status_word

        inb = symm.empty(cap_rows * dim, dtype=torch.bfloat16, device=self.device)
        outb = symm.empty(cap_rows * dim, dtype=torch.bfloat16, device=self.device)
        flags = symm.empty(64, dtype=torch.int32, device=self.device)
        flags.zero_()
        # one 16-byte record per received row: (sender rank + 1, the row's flat (token, slot) index, 0, 0)
        tagb = symm.empty(cap_rows * 8, dtype=torch.bfloat16, device=self.device)
        tagb.zero_()  # each dispatch clears the records it has consumed, so the buffer is clean between exchanges
        # per-expert row counts of every rank, double buffered by call parity: int32 [2][8][slots]
        from mintext_b200.ops._ext import ext

        countb = symm.empty(2 * 8 * int(ext().ep_count_slots()), dtype=torch.int32, device=self.device)
        countb.zero_()
        h_cnt = symm.rendezvous(countb, self.group)
        h_in, h_out, h_fl, h_tag = (symm.rendezvous(t, self.group) for t in (inb, outb, flags, tagb))
        self._bufs = {
            "cap": cap_rows, "dim": dim, "in": inb.view(cap_rows, dim), "out": outb.view(cap_rows, dim),
            "in_ptrs": [int(p) for p in h_in.buffer_ptrs], "out_ptrs": [int(p) for p in h_out.buffer_ptrs],
            "flag_ptrs": [int(p) for p in h_fl.buffer_ptrs], "handles": (h_in, h_out, h_fl, h_tag), "flags": flags,
            "tag": tagb.view(cap_rows, 8), "tag_ptrs": [int(p) for p in h_tag.buffer_ptrs],
            "counts": countb, "count_ptrs": [int(p) for p in h_cnt.buffer_ptrs], "h_cnt": h_cnt,
            "out_ptr_table": torch.tensor([int(p) for p in h_out.buffer_ptrs], dtype=torch.int64, device=self.device),
            "in_ptr_table": torch.tensor([int(p) for p in h_in.buffer_ptrs], dtype=torch.int64, device=self.device),
        }
        self.overflow = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.seq = 0
        self.calls = 0
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        status_word(self.device)
        return self._bufs

    def barrier(self) -> None:
        from mintext_b200.ops._ext import ext, status_word

        self.seq += 1
        ext().symm_barrier(self._bufs["flag_ptrs"], self.rank, self.seq, status_word(self.device))

    def dropped_counter(self) -> torch.Tensor:
        """Device counter of routed rows dropped because a destination's receive capacity was exhausted."""
        if self._dropped is None:
            self._dropped = torch.zeros(1, dtype=torch.int64, device=self.device)
        return self._dropped

    def dropped_rows(self, reset: bool = True) -> int:
        """Routed rows dropped for lack of receive capacity since the last call (synchronises)."""
        n = 0 if self._dropped is None else int(self._dropped.item())
        if reset and self._dropped is not None:
            self._dropped.zero_()
        return n

    def check_overflow(self) -> None:
        """Raise if a push kernel met a row beyond the receive capacity that the plan had not already dropped."""
        if self.overflow is not None and int(self.overflow.item()) != 0:
            self.overflow.zero_()
            raise RuntimeError("expert-parallel dispatch overflowed a receive buffer; raise moe capacity_factor")


# ------------------------------------------------------------------------------------------ differentiable collectives
class _AllGatherRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        n = dist.get_world_size(group)
        out = [torch.empty_like(x) for _ in range(n)]
        dist.all_gather(out, x.contiguous(), group=group)
        return torch.cat(out, dim=0)

    @staticmethod
    def backward(ctx, g):
        n, r = dist.get_world_size(ctx.group), dist.get_rank(ctx.group)
        g = g.contiguous()
        dist.all_reduce(g, group=ctx.group)
        per = g.shape[0] // n
        return g[r * per:(r + 1) * per], None


class _ReduceScatterRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        n, r = dist.get_world_size(group), dist.get_rank(group)
        x = x.contiguous().clone()
        dist.all_reduce(x, group=group)
        per = x.shape[0] // n
        return x[r * per:(r + 1) * per].clone()

    @staticmethod
    def backward(ctx, g):
        n = dist.get_world_size(ctx.group)
        out = [torch.empty_like(g) for _ in range(n)]
        dist.all_gather(out, g.contiguous(), group=ctx.group)
        return torch.cat(out, dim=0), None


def experts_forward_collective(ep: ExpertParallel, x, topk_idx, topk_w, gate_up_local, down_local, act: str,
                               num_experts: int, dtype):
    """All-gather tokens and routing, serve the slots owned by the local experts, reduce-scatter the outputs."""
    from mintext_b200 import kernels
    from mintext_b200.ops import functional as F

    lo, hi = ep.local_expert_range(num_experts)
    xa = _AllGatherRows.apply(x, ep.group)
    ia = _AllGatherRows.apply(topk_idx, ep.group)
    wa = _AllGatherRows.apply(topk_w, ep.group)
    mine = (ia >= lo) & (ia < hi)                      # [ep*N, K]
    tok, slot = torch.nonzero(mine, as_tuple=True)     # host sync: acceptable on the baseline path
    e_local = ia[tok, slot] - lo
    order = torch.argsort(e_local, stable=True)
    tok, slot, e_local = tok[order], slot[order], e_local[order]
    sizes = torch.bincount(e_local, minlength=hi - lo)
    rows = xa.index_select(0, tok)
    h = kernels.grouped_matmul_vjp(rows, gate_up_local.to(dtype), sizes)
    h = F.gated_act(h, act)
    y = kernels.grouped_matmul_vjp(h, down_local.to(dtype), sizes)
    y = y * wa[tok, slot].to(y.dtype)[:, None]
    partial = torch.zeros_like(xa).index_add(0, tok, y)
    return _ReduceScatterRows.apply(partial, ep.group)


# ------------------------------------------------------------------------------------------ peer-memory path
def _plan(ep: ExpertParallel, topk_idx: torch.Tensor, topk_w: torch.Tensor, num_experts: int, cap: int, dim: int):
    """Device-side routing plan, in flat (token, slot) order: for every local entry its destination rank and its
    row in that rank's expert-contiguous, 128-padded buffer, plus the padded offsets of this rank's own experts.
    The per-expert counts and the stable rank of every entry inside its expert come from the counting-sort kernel;
    the ranks exchange their counts by peer stores into a small symmetric table, and one kernel derives the plan
    from it.  No host synchronisation, no library collective.

    Capacity: a destination rank holds at most ``cap`` rows.  Rows that would land beyond it are dropped (they
    contribute nothing to the token's output and receive no gradient, as in capacity-factor routing): the sender
    marks them with rank -1 / home position -1, and every rank truncates its own expert offsets at ``cap``, so no
    kernel on either side ever indexes past a buffer."""
    from mintext_b200.ops import moe as moe_ops
    from mintext_b200.ops._ext import ext

    N, K = topk_idx.shape
    E, R = num_experts, ep.size
    flat = topk_idx.reshape(-1).contiguous()
    counts, off_l, pos_l, _ = ext().moe_sort(flat, E, moe_ops.capacity(flat.numel(), E))
    b = ep.buffers(cap, dim)
    parity = ep.calls & 1
    ep.calls += 1
    ext().ep_push_counts(counts, b["count_ptrs"], ep.rank, parity)
    # every rank's counts are in every table; also: no peer still uses this rank's buffers from an earlier exchange
    ep.barrier()
    w = topk_w.detach().reshape(-1).float().contiguous()
    dst_rank, dst_pos, home_pos, off_local, tags = ext().ep_plan(flat, pos_l, off_l, w, b["counts"], parity, ep.rank, R,
                                                                 E, cap, K, ep.dropped_counter())
    return {"dst_rank": dst_rank, "dst_pos": dst_pos, "rank_flat": dst_rank, "pos_flat": dst_pos, "home_pos": home_pos,
            "off_local": off_local, "send_tags": tags, "cap": cap, "N": N, "K": K}


def _src_token(plan) -> torch.Tensor:
    """Token row of every flat (token, slot) entry (only the unfused fallbacks need it as a tensor)."""
    if "src_token" not in plan:
        idx = torch.arange(plan["N"] * plan["K"], device=plan["dst_pos"].device)
        plan["src_token"] = torch.div(idx, plan["K"], rounding_mode="floor")
    return plan["src_token"]


def _dispatch_rows(x, ep, plan):
    """Forward half of the dispatch.  Every rank publishes its tokens in its symmetric buffer and sends each expert
    rank one 16-byte record per routed (token, slot): (sender + 1, flat (token, slot) index, token row, routing
    weight).  The expert rank then pulls the rows it was promised with one table-driven gather that also lays them
    out expert-contiguous and 128-padded (zero rows in the padding).  Returns those rows; the addresses derived from
    the records stay in the plan (``row_src``: where a row came from, ``row_dst``: where its result goes back to,
    ``row_scale``: its routing weight).  The barrier that opens the exchange is the one inside :func:`_plan`."""
    from mintext_b200.ops._ext import ext

    N, D = x.shape
    b = ep.buffers(plan["cap"], D)
    b["in"][:N].copy_(x)
    ext().ep_push_rows(plan["send_tags"].view(torch.bfloat16), plan["dst_rank"], plan["dst_pos"], b["tag_ptrs"], b["cap"],
                       ep.overflow)
    ep.barrier()  # records have landed, tokens are published
    got = b["tag"][: plan["cap"]].view(torch.int32).clone()
    b["tag"].zero_()  # cleared before this rank passes the closing barrier, i.e. before any peer's next records
    plan["row_src"], plan["row_dst"], plan["row_scale"] = ext().ep_resolve(got, b["in_ptrs"], b["out_ptrs"], D * 2)
    rows = torch.empty(plan["cap"], D, device=x.device, dtype=x.dtype)
    ext().ep_gather_rows(rows, plan["row_src"], torch.empty(0, device=x.device))
    ep.barrier()  # every rank has its rows: the token buffers may be reused
    return rows


class _Dispatch(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, ep, plan):
        ctx.ep, ctx.plan, ctx.n = ep, plan, x.shape[0]
        return _dispatch_rows(x, ep, plan)

    @staticmethod
    def backward(ctx, d_rows):
        from mintext_b200.ops._ext import ext

        ep, plan = ctx.ep, ctx.plan
        b = ep.buffers(plan["cap"], d_rows.shape[1])
        b["out"][: plan["cap"]].copy_(d_rows)
        ep.barrier()
        pulled = torch.empty(plan["dst_rank"].numel(), d_rows.shape[1], device=d_rows.device, dtype=d_rows.dtype)
        ext().ep_pull_rows(pulled, plan["dst_rank"], plan["dst_pos"], b["out_ptrs"], b["cap"])
        ep.barrier()
        dx = torch.zeros(ctx.n, d_rows.shape[1], device=d_rows.device, dtype=torch.float32)
        dx.index_add_(0, _src_token(plan), pulled.float())
        return dx.to(d_rows.dtype), None, None


class _Combine(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y_p, w, ep, plan):
        from mintext_b200.ops._ext import ext

        b = ep.buffers(plan["cap"], y_p.shape[1])
        b["out"][: plan["cap"]].copy_(y_p)
        ep.barrier()
        N, K = plan["N"], plan["K"]
        picked = torch.empty(N * K, y_p.shape[1], device=y_p.device, dtype=y_p.dtype)
        ext().ep_pull_rows(picked, plan["rank_flat"], plan["pos_flat"], b["out_ptrs"], b["cap"])
        ep.barrier()
        ctx.save_for_backward(picked, w)
        ctx.ep, ctx.plan = ep, plan
        return torch.einsum("nkd,nk->nd", picked.view(N, K, -1), w.to(picked.dtype))

    @staticmethod
    def backward(ctx, dy):
        from mintext_b200.ops._ext import ext

        picked, w = ctx.saved_tensors
        ep, plan = ctx.ep, ctx.plan
        N, K = plan["N"], plan["K"]
        d_picked = (dy[:, None, :] * w.to(dy.dtype)[:, :, None]).reshape(N * K, -1).contiguous()
        dw = torch.einsum("nkd,nd->nk", picked.view(N, K, -1).float(), dy.float()).to(w.dtype)
        b = ep.buffers(plan["cap"], dy.shape[1])
        b["in"].zero_()
        ep.barrier()
        ext().ep_push_rows(d_picked, plan["rank_flat"], plan["pos_flat"], b["in_ptrs"], b["cap"], ep.overflow)
        ep.barrier()
        return b["in"][: plan["cap"]].clone(), dw, None, None


def _grouped_plain(x, w, off, w_is_ekn: bool, fp8: bool):
    """Grouped product that stays on this rank (no row scatter): ``x @ w[e]`` (``w_is_ekn``) or ``x @ w[e]^T``; in
    block-scaled FP8 when asked for and the shapes allow it, else bf16."""
    from mintext_b200.ops import moe as moe_ops
    from mintext_b200.ops._ext import ext, status_word

    e, st = ext(), status_word(x.device)
    if fp8 and moe_ops.mxfp8_grouped_path(x, w):
        xq, xs, _, _ = e.mxfp8_quantize(x, True, False, False, False)
        if w_is_ekn:   # contraction over K: the kernel wants [E, N, K]
            _, _, wq, ws = e.mxfp8_quantize_stack(w, False, True)
        else:          # contraction over N: w as stored is [E, K(out), N(contraction)]
            wq, ws, _, _ = e.mxfp8_quantize_stack(w, True, False)
        return e.grouped_gemm_mxfp8(xq, xs, wq, ws, off, st)
    y = torch.empty(x.shape[0], w.shape[2] if w_is_ekn else w.shape[1], device=x.device, dtype=torch.bfloat16)
    e.grouped_gemm(x, w, y, off, w_is_ekn, st)
    return y


class _GroupedCombine(torch.autograd.Function):
    """Down projection of the local experts fused with the combine all-to-all: ONE kernel multiplies the expert
    tiles and writes every output row from its epilogue straight into the home rank's receive buffer over NVLink
    (csrc/gemm/grouped_bf16_2cta.cu, SCATTER), so the transfer overlaps the remaining tiles; the home rank then
    reduces its K rows per token with the routing weights.  Backward: push of the weighted output gradients to the
    expert ranks, then the grouped data- and weight-gradient GEMMs."""

    @staticmethod
    def forward(ctx, h, w, topk_w, main_grad, ep, plan, fp8=False):
        from mintext_b200.ops._ext import ext, status_word

        ctx.fp8 = fp8
        D = w.shape[2]
        N, K = plan["N"], plan["K"]
        b = ep.buffers(plan["cap"], D)
        # no barrier in front: a rank's last read of its receive buffer (the previous exchange) precedes, in stream
        # order, its arrival at this layer's dispatch barriers, which every peer has passed before it gets here
        ext().grouped_gemm_scatter(h, w, plan["row_dst"], plan["off_local"], True, status_word(h.device))
        ep.fused_combines = getattr(ep, "fused_combines", 0) + 1
        ep.barrier()  # every rank's rows have landed
        picked = b["out"][: N * K].clone()
        ctx.save_for_backward(h, w, picked, topk_w)
        ctx.ep, ctx.plan, ctx.main_grad = ep, plan, main_grad
        # weighted sum of each token's K adjacent rows (row-reduction kernel of the single-GPU path, identity index)
        out, _ = ext().moe_combine_rows(picked, plan["home_pos"], topk_w.detach().float().contiguous(), N, K, True, None)
        return out

    @staticmethod
    def backward(ctx, dy):
        from mintext_b200.ops._ext import ext, status_word

        h, w, picked, topk_w = ctx.saved_tensors
        ep, plan = ctx.ep, ctx.plan
        N, K = plan["N"], plan["K"]
        st = status_word(h.device)
        D = dy.shape[1]
        dy = dy.contiguous()
        _, dtw = ext().moe_combine_rows(picked, plan["home_pos"], None, N, K, False, dy)
        dtw = dtw.to(topk_w.dtype)
        b = ep.buffers(plan["cap"], D)
        # the expert ranks pull dy[token] * routing weight for each of their rows (weights came with the dispatch
        # records), so the weighted [N*K, D] gradient is never materialised on the home rank.  The token buffer is
        # free: its last readers (the previous exchange) finished before that exchange's closing barrier.
        b["in"][:N].copy_(dy)
        ep.barrier()  # every rank's output gradient is published
        dy_p = torch.empty(plan["cap"], D, device=dy.device, dtype=dy.dtype)
        ext().ep_gather_rows(dy_p, plan["row_src"], plan["row_scale"])
        ep.barrier()  # all pulls done: the buffers may be reused
        dh = _grouped_plain(dy_p, w, plan["off_local"], False, ctx.fp8)
        dw = None
        if ctx.main_grad is not None:
            ext().grouped_wgrad(h, dy_p, ctx.main_grad.view(w.shape), plan["off_local"], True, st)
        else:
            dwf = torch.zeros(w.shape, device=w.device, dtype=torch.float32)
            ext().grouped_wgrad(h, dy_p, dwf, plan["off_local"], False, st)
            dw = dwf.to(w.dtype)
        return dh, dw, dtw, None, None, None, None


class _DispatchGrouped(torch.autograd.Function):
    """Dispatch + first expert projection.  Forward: peer-store dispatch, then the grouped GEMM.  Backward: the
    grouped data-gradient GEMM fused with the dispatch-gradient all-to-all - its epilogue writes every gradient row
    straight back to the rank the token came from (same SCATTER kernel as the fused combine)."""

    @staticmethod
    def forward(ctx, x, w, main_grad, ep, plan, fp8=False):
        rows = _dispatch_rows(x, ep, plan)
        y = _grouped_plain(rows, w, plan["off_local"], True, fp8)
        ctx.save_for_backward(rows, w)
        ctx.ep, ctx.plan, ctx.main_grad, ctx.n = ep, plan, main_grad, x.shape[0]
        return y

    @staticmethod
    def backward(ctx, dy):
        from mintext_b200.ops._ext import ext, status_word

        rows, w = ctx.saved_tensors
        ep, plan = ctx.ep, ctx.plan
        st = status_word(rows.device)
        dy = dy.contiguous()
        D = rows.shape[1]
        dw = None
        if ctx.main_grad is not None:
            ext().grouped_wgrad(rows, dy, ctx.main_grad.view(w.shape), plan["off_local"], True, st)
        else:
            dwf = torch.zeros(w.shape, device=w.device, dtype=torch.float32)
            ext().grouped_wgrad(rows, dy, dwf, plan["off_local"], False, st)
            dw = dwf.to(w.dtype)
        b = ep.buffers(plan["cap"], D)
        # rows go home to their flat (token, slot) position, so a token's K gradient rows are adjacent and the
        # reduction over slots needs no atomics
        # (no barrier in front, as in the fused combine: the combine-gradient barriers of this layer lie in between)
        ext().grouped_gemm_scatter(dy, w, plan["row_dst"], plan["off_local"], False, st)  # dy @ w[e]^T, rows sent home
        ep.barrier()
        N, K = plan["N"], plan["K"]
        # sum of each token's K adjacent gradient rows; rows of dropped slots were never written and are skipped
        dx, _ = ext().moe_combine_rows(b["out"][: N * K], plan["home_pos"], None, N, K, True, None)
        return dx, dw, None, None, None, None


def _fused_combine_ok(ep: ExpertParallel, plan, down_local) -> bool:
    import os

    from mintext_b200.ops._ext import ext

    return (os.environ.get("MT_EP_FUSED_COMBINE", "1") != "0" and hasattr(ext(), "grouped_gemm_scatter")
            and down_local.dtype == torch.bfloat16 and down_local.shape[2] > 128 and down_local.shape[2] % 8 == 0
            and down_local.shape[0] <= 256 and plan["N"] * plan["K"] <= plan["cap"])


def experts_forward_peer(ep: ExpertParallel, x, topk_idx, topk_w, gate_up_local, down_local, act: str,
                         num_experts: int, fp8: bool = False):
    """``fp8``: the expert GEMMs that stay on the rank (gate/up forward, down data gradient) run block-scaled; the two
    fused with a row scatter over NVLink (down forward, gate/up data gradient) stay bf16."""
    from mintext_b200.ops import functional as F
    from mintext_b200.ops import moe as moe_ops

    N, K = topk_idx.shape
    El = num_experts // ep.size
    cap = moe_ops.capacity(int(ep.capacity_factor * N * K), El)
    plan = _plan(ep, topk_idx, topk_w, num_experts, cap, x.shape[1])
    fused = _fused_combine_ok(ep, plan, down_local)
    if fused and x.shape[1] > 128 and x.dtype == torch.bfloat16:
        h = _DispatchGrouped.apply(x.contiguous(), gate_up_local, getattr(gate_up_local, "main_grad", None), ep, plan,
                                   fp8)
    else:
        rows = _Dispatch.apply(x, ep, plan)
        h = moe_ops.grouped_padded(rows, gate_up_local, plan["off_local"], None, fp8)
    h = F.gated_act(h, act)
    if fused:
        return _GroupedCombine.apply(h.contiguous(), down_local, topk_w, getattr(down_local, "main_grad", None), ep, plan,
                                     fp8)
    y = moe_ops.grouped_padded(h, down_local, plan["off_local"], None, fp8)
    return _Combine.apply(y, topk_w, ep, plan)
