"""Vocabulary-parallel embedding and output head for a tensor-parallel group.

The reference maps the ``vocab`` axis of the embedding table and of the output projection to the ``tensor`` mesh axis
(mintext/config.py:83-89; mintext/models/base.py:199-203,231-239), which leaves the compiler to partition the lookup
and the softmax.  Here the residual stream of a tensor-parallel group is sharded over tokens, so the two ends of the
model are written out:

* embedding: every rank holds rows ``[v_lo, v_hi)`` of the table.  The group's token ids are gathered (a few
  kilobytes), each rank looks up the ids that fall into its rows (zeros elsewhere), and a reduce-scatter over tokens
  leaves every rank with the embeddings of its own token shard.  Exactly one rank contributes a non-zero row per
  token, so the sum is exact in any dtype.
* output head + cross-entropy: the hidden states are gathered over the group, every rank forms the logits of its
  vocabulary slice ``[N, V/t]`` (in token chunks, never all at once), and three small reductions over the group
  complete the softmax: the row maximum, then the sum of exponentials, the target logit and the sum of logits
  (label smoothing) in one call.  The backward pass recomputes the chunk's logits, forms ``d logits`` in place and
  reduces ``d hidden`` back to token shards with one reduce-scatter.

Loss convention: every rank returns the per-token losses of its own token shard, as the unsharded head does, so the
trainer's normalisation does not change.

Enabled with ``tp_vocab_parallel: true``; it trades one gather and one reduce-scatter of ``[N, D]`` per end for
``1/t`` of the two largest matrices of a small-hidden / large-vocabulary model.  The collectives are the group's
library calls and the GEMMs plain matmuls: this path is about memory, the unsharded head keeps the fused
projection + loss kernel.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from mintext_b200.parallel.tp import TensorParallel, _reduce_scatter, reduce_scatter_tokens


def _gather_rows(x: torch.Tensor, group) -> torch.Tensor:
    """``[n, ...] -> [t*n, ...]``, rank 0's rows first (no gradient)."""
    n = dist.get_world_size(group)
    out = torch.empty((n * x.shape[0],) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    dist.all_gather_into_tensor(out, x.contiguous(), group=group)
    return out


def shard_vocab_rows(full: torch.Tensor, tp: TensorParallel, dim: int) -> torch.Tensor:
    lo, hi = tp.shard(full.shape[dim], "vocab_size")
    return full.narrow(dim, lo, hi - lo).clone().contiguous()


def embedding(table_local: torch.Tensor, tokens_local: torch.Tensor, tp: TensorParallel, dtype,
              scale: float | None = None) -> torch.Tensor:
    """``tokens_local`` ``[1, n]`` (this rank's token shard) -> ``[1, n, D]`` from the rank's table rows
    ``[V/t, D]``.  Differentiable in ``table_local``."""
    vl = table_local.shape[0]
    v_lo = tp.rank * vl
    ids = _gather_rows(tokens_local.reshape(-1), tp.group) - v_lo
    mine = (ids >= 0) & (ids < vl)
    rows = table_local[ids.clamp(0, vl - 1)].to(dtype) * mine[:, None].to(dtype)
    x = reduce_scatter_tokens(rows, tp)
    if scale is not None:
        x = x * scale
    return x.view(tokens_local.shape[0], tokens_local.shape[1], -1)


class _LinearCrossEntropy(torch.autograd.Function):
    @staticmethod
    def forward(ctx, h, w, targets, tp, weight_is_vd, label_smoothing, z_loss_weight, softcap, chunks):
        group = tp.group
        hf = _gather_rows(h, group)                      # [N, D]
        tf = _gather_rows(targets.reshape(-1), group)    # [N]
        N = hf.shape[0]
        vl = w.shape[0] if weight_is_vd else w.shape[1]
        V, v_lo = vl * tp.size, tp.rank * vl
        wt = (w if weight_is_vd else w.t()).to(hf.dtype)  # [V/t, D]
        rel = tf - v_lo
        mine = (rel >= 0) & (rel < vl)
        relc = rel.clamp(0, vl - 1)
        mx = torch.empty(N, dtype=torch.float32, device=hf.device)
        part = torch.empty(3, N, dtype=torch.float32, device=hf.device)  # sum exp(l - local max), target logit, sum l
        step = -(-N // max(int(chunks), 1))
        for a in range(0, N, step):
            sl = slice(a, min(a + step, N))
            lg = (hf[sl] @ wt.t()).float()
            if softcap is not None:
                lg = torch.tanh(lg / softcap) * softcap
            m = lg.max(dim=-1).values
            mx[sl] = m
            part[0, sl] = torch.exp(lg - m[:, None]).sum(-1)
            part[1, sl] = lg.gather(-1, relc[sl, None]).squeeze(-1) * mine[sl].float()
            part[2, sl] = lg.sum(-1)
        gmx = mx.clone()
        dist.all_reduce(gmx, op=dist.ReduceOp.MAX, group=group)
        part[0] *= torch.exp(mx - gmx)
        dist.all_reduce(part, group=group)
        lse = gmx + torch.log(part[0])
        z = z_loss_weight * lse * lse
        loss = lse - (1.0 - label_smoothing) * part[1] - label_smoothing * part[2] / V + z
        n = h.shape[0]
        own = slice(tp.rank * n, (tp.rank + 1) * n)
        ctx.save_for_backward(hf, wt, lse, relc, mine)
        ctx.meta = (tp, weight_is_vd, label_smoothing, z_loss_weight, softcap, step, V, h.dtype, w.dtype)
        z_own = z[own].clone()
        ctx.mark_non_differentiable(z_own)
        return loss[own].clone(), z_own

    @staticmethod
    def backward(ctx, g_loss, _g_z):
        hf, wt, lse, relc, mine = ctx.saved_tensors
        tp, weight_is_vd, ls, zw, softcap, step, V, h_dtype, w_dtype = ctx.meta
        N = hf.shape[0]
        gf = _gather_rows(g_loss.float().reshape(-1), tp.group)  # d(sum of the ranks' losses) / d(per-token loss)
        dh = torch.empty_like(hf)
        dwt = torch.zeros(wt.shape, dtype=torch.float32, device=wt.device)
        rows = torch.arange(N, device=hf.device)
        for a in range(0, N, step):
            sl = slice(a, min(a + step, N))
            lg = (hf[sl] @ wt.t()).float()
            if softcap is not None:
                th = torch.tanh(lg / softcap)
                lg = th * softcap
            d = torch.exp(lg - lse[sl, None]) * (1.0 + 2.0 * zw * lse[sl])[:, None]
            if ls:
                d -= ls / V
            r = rows[: sl.stop - sl.start][mine[sl]]
            d[r, relc[sl][mine[sl]]] -= 1.0 - ls
            d *= gf[sl, None]
            if softcap is not None:
                d *= 1.0 - th * th
            dc = d.to(hf.dtype)
            dh[sl] = dc @ wt
            dwt += (dc.t() @ hf[sl]).float()
        dh_own = _reduce_scatter(dh, tp.group)
        dw = dwt if weight_is_vd else dwt.t()
        return dh_own.to(h_dtype), dw.to(w_dtype).contiguous(), None, None, None, None, None, None, None


def linear_cross_entropy(h: torch.Tensor, w_local: torch.Tensor, targets: torch.Tensor, tp: TensorParallel,
                         weight_is_vd: bool, label_smoothing: float = 0.0, z_loss_weight: float = 0.0,
                         softcap: float | None = None, chunks: int = 1):
    """Per-token ``(loss incl. z-loss, z-loss)`` of this rank's token shard: ``h`` ``[n, D]``, ``targets`` ``[n]``,
    ``w_local`` the rank's vocabulary slice (``[V/t, D]`` if ``weight_is_vd`` else ``[D, V/t]``).  Same definition
    as ``ops/oracle.py::cross_entropy`` on the logits ``softcap(h @ W)``."""
    return _LinearCrossEntropy.apply(h, w_local, targets, tp, bool(weight_is_vd), float(label_smoothing),
                                     float(z_loss_weight), softcap, int(chunks))
