"""B200 training engine: flat parameter / gradient storage, sharded fused optimizer, device-timed steps.

Memory plan (sized for 180 GB of HBM3e per GPU): every rank keeps the *whole* bf16 compute copy of the
parameters resident in one flat buffer (a 1 B model is 2.5 GB, an 8 B model 16 GB), so forward and backward
never wait for a parameter gather.  What is sharded ``1/N`` over the ``data x fsdp`` ranks is everything that is
only touched once per step: the fp32 master weights and both Adam moments.  Gradients accumulate in one flat
fp32 buffer that the wgrad GEMM epilogues add into directly (no per-parameter ``.grad`` tensors, no cast pass).

One optimizer step is then
  1. reduce-scatter of the flat fp32 gradient (each rank ends up with the sum of its shard),
  2. the global gradient norm from per-shard sums of squares (one scalar all-reduce),
  3. the fused AdamW kernel on the shard (clip factor, moments, master update, bf16 cast in one pass),
  4. all-gather of the updated bf16 shard into every rank's compute buffer.
With ``fused_collectives`` steps 1 and 3+4 run as this repository's peer-memory kernels (pull-reduce over
NVLink, update, push to every peer); otherwise they are NCCL reduce-scatter / all-gather around the same AdamW
kernel.  Small fp32 parameters (norm scales, gate biases ...) are replicated and updated redundantly from
all-reduced gradients.

The rule for which GPU holds which batch rows: the global batch is split evenly over all ranks of the
``data`` and ``fsdp`` axes (true FSDP, unlike the reference, which replicates the batch over ``fsdp``).
"""

from __future__ import annotations

import json
import os
from dataclasses import dataclass

import torch
import torch.distributed as dist

from mintext_b200.ops._ext import check_status, ext
from mintext_b200.optim.optimizer import create_lr_schedule, weight_decay_mask
from mintext_b200.utils.profiling import nvtx_range

_ALIGN = 64  # elements; keeps every parameter view 128-byte aligned for TMA


@dataclass
class _Slot:
    name: str
    param: torch.nn.Parameter
    offset: int
    numel: int
    bucket: int = 0  # index into the engine's bucket list (sharded group only)


class FlatGroup:
    """Parameters of one kind laid out back to back in flat buffers."""

    def __init__(self, slots: list[_Slot], total: int):
        self.slots = slots
        self.total = total


def _round_up(x: int, m: int) -> int:
    return (x + m - 1) // m * m


def bucket_of(name: str) -> int:
    """Gradient bucket of a parameter: decoder layer ``i`` is bucket ``i + 1``; everything else (embedding, output
    head, final norm) is bucket 0, whose gradients are complete only when the whole backward pass is."""
    parts = name.split(".")
    if len(parts) > 2 and parts[0] == "layers" and parts[1].isdigit():
        return int(parts[1]) + 1
    return 0


def plan_buckets(sizes: list[tuple[int, int]], world: int, align: int = _ALIGN, quantum: int = 1024):
    """Lay parameters out bucket by bucket.  ``sizes`` lists ``(bucket id, numel)`` per parameter in model order.
    Returns ``(offsets, buckets, total)``: the flat offset of every parameter, and per bucket (ascending id)
    ``(bucket id, flat offset, length)`` with every length a multiple of ``world * quantum``, so that each rank owns
    one contiguous, vector-aligned ``length / world`` slice of every bucket."""
    ids = sorted({b for b, _ in sizes})
    cursor = {b: 0 for b in ids}
    rel = []
    for b, n in sizes:
        rel.append((b, cursor[b]))
        cursor[b] = _round_up(cursor[b] + n, align)
    buckets, start, base = [], {}, 0
    for b in ids:
        length = _round_up(max(cursor[b], 1), world * quantum)
        buckets.append((b, base, length))
        start[b] = base
        base += length
    return [start[b] + off for b, off in rel], buckets, base


class TrainEngine:
    """Owns the device copies of a model's parameters and runs optimizer steps on them.

    ``model`` must have been built on the CPU in ``weight_dtype`` (fp32); the engine moves it to ``device``,
    re-homes every parameter into the flat buffers and keeps the fp32 values as (sharded) master weights.
    """

    def __init__(self, model: torch.nn.Module, config, device: torch.device | str = "cuda", group=None,
                 local_reduce_group=None, expert_reduce_group=None):
        """``group``: ranks over which replicated parameters are reduced and the optimizer state is sharded
        (default: all ranks).  ``local_reduce_group``: ranks that hold *the same* slice of the expert- or
        tensor-parallel parameters (their data-parallel replicas); None when every rank's slice is unique.
        ``expert_reduce_group``: given when tensor and expert parallelism are combined, where the two kinds of
        slices have different replicas (tensor slices: the ranks of the same tensor coordinate; expert slices: the
        ranks at the same expert position, across the tensor axis): then ``local_reduce_group`` serves the tensor
        slices and this group the expert slices."""
        self.config = config
        self.local_reduce_group = local_reduce_group
        self.local_reduce_size = dist.get_world_size(local_reduce_group) if local_reduce_group is not None else 1
        self.expert_reduce_group = expert_reduce_group
        self.expert_reduce_size = dist.get_world_size(expert_reduce_group) if expert_reduce_group is not None else 1
        self.model = model
        self.device = torch.device(device)
        self.group = group
        self.world = dist.get_world_size(group) if (dist.is_available() and dist.is_initialized()) else 1
        self.rank = dist.get_rank(group) if self.world > 1 else 0
        self.schedule = create_lr_schedule(config)
        self.step_count = 0
        self.compute_dtype = config.torch_dtype
        self._build_storage()
        self.use_fused = bool(config.fused_collectives) and self.world > 1 and config.optimizer == "adamw"
        self._comm = None
        if self.use_fused and self._use_symmetric_optimizer_comm():
            try:
                from mintext_b200.parallel.symm import SymmetricOptimizerComm

                self._comm = SymmetricOptimizerComm(self)
            except Exception as e:  # fall back to the NCCL composition, loudly
                import logging

                logging.getLogger(__name__).warning("peer-memory optimizer path unavailable (%s); using NCCL", e)
                self.use_fused = False
        self._muon_comm = None
        if self.use_muon and self.world > 1 and bool(config.fused_collectives) and self.param_flat is not None:
            try:
                from mintext_b200.parallel.symm import MuonPublishComm

                self._muon_comm = MuonPublishComm(self)
            except Exception as e:  # fall back to the NCCL all-gather, loudly
                import logging

                logging.getLogger(__name__).warning("peer-memory Muon publication unavailable (%s); using NCCL", e)
        self._sumsq = torch.zeros(1, device=self.device, dtype=torch.float32)
        self._sumsq_shard = torch.zeros(1, device=self.device, dtype=torch.float32)
        self._clip = torch.ones(1, device=self.device, dtype=torch.float32)
        self.kernel_launches = 0
        self._flat_cleared_by_pull = False
        self._pulled: set[int] = set()   # buckets whose reduction has been issued in this step
        self._late: set[int] = set()     # ... and that received further gradients afterwards
        self._slots_of_bucket = None
        self._has_tp_replicated = None

    sharded_params = False  # True in the subclass that shards layer weights and gradients (parallel/fsdp.py)

    def _use_symmetric_optimizer_comm(self) -> bool:
        return True

    # ------------------------------------------------------------------ storage
    def _build_storage(self) -> None:
        cfg = self.config
        dev = self.device
        big: list[_Slot] = []
        small: list[_Slot] = []
        exp: list[_Slot] = []
        off_e = 0
        frozen: list[tuple[str, torch.nn.Parameter]] = []
        off_b = off_s = 0
        for name, p in self.model.named_parameters():
            if not p.requires_grad:
                frozen.append((name, p))
                continue
            is_big = p.dim() >= 2 and p.numel() >= 4096 and "conv_weight" not in name
            if (getattr(p, "expert_parallel", False) or getattr(p, "tensor_parallel", False)) \
                    and self.compute_dtype == torch.bfloat16:
                exp.append(_Slot(name, p, off_e, p.numel()))  # this rank's experts: local, not sharded
                off_e = _round_up(off_e + p.numel(), _ALIGN)
            elif is_big and self.compute_dtype == torch.bfloat16:
                big.append(_Slot(name, p, off_b, p.numel()))
                off_b = _round_up(off_b + p.numel(), _ALIGN)
            else:
                small.append(_Slot(name, p, off_s, p.numel()))
                off_s = _round_up(off_s + p.numel(), _ALIGN)
        self.use_muon = cfg.optimizer == "muon"
        # Flat layout of the sharded group.  One bucket per decoder layer (plus one for the rest), each split 1/N
        # over the ranks: a rank's optimizer shard is the concatenation of its slice of every bucket, and a bucket's
        # gradients can be reduced as soon as the backward pass has left its layer.  Muon keeps whole matrices on
        # one rank instead (one bucket, bin-packed).
        if self.use_muon and self.world > 1 and big:
            total_b = self._matrix_aligned_layout(big)
            buckets = [(0, 0, total_b)]
        elif self.compute_dtype == torch.bfloat16 and big and self.world > 1:
            offs, buckets, total_b = plan_buckets([(bucket_of(s.name), s.numel) for s in big], self.world)
            for s, o in zip(big, offs):
                s.offset = o
        else:
            total_b = _round_up(max(off_b, 1), self.world * 1024)
            buckets = [(0, 0, total_b)]
        self.big = FlatGroup(big, total_b)
        self.small = FlatGroup(small, _round_up(max(off_s, 1), _ALIGN))
        self.shard_size = total_b // self.world
        # (bucket id, flat range of this rank's slice, offset of the slice in the rank's shard arrays)
        self.segments: list[tuple[int, int, int, int]] = []
        local = 0
        for bid, boff, blen in buckets:
            sl = blen // self.world
            self.segments.append((bid, boff + self.rank * sl, boff + (self.rank + 1) * sl, local))
            local += sl
        self.buckets = buckets
        self._bucket_index = {bid: i for i, (bid, _, _) in enumerate(buckets)}

        self._alloc_sharded_group(big, buckets, total_b)

        # expert-parallel parameters: every rank owns its experts outright (compute copy, master, moments, grads)
        self._exp_split = None
        if exp and self.expert_reduce_group is not None:
            # tensor slices first, expert slices behind them: two contiguous ranges with their own replica groups
            exp.sort(key=lambda sl: bool(getattr(sl.param, "expert_parallel", False)))
            off_e = 0
            for sl in exp:
                if self._exp_split is None and getattr(sl.param, "expert_parallel", False):
                    self._exp_split = off_e
                sl.offset = off_e
                off_e = _round_up(off_e + sl.numel, _ALIGN)
            if self._exp_split is None:
                self._exp_split = off_e
        self.exp = FlatGroup(exp, _round_up(max(off_e, 4), _ALIGN))
        if exp:
            self.exp_master = torch.zeros(self.exp.total, device=dev, dtype=torch.float32)
            self.exp_param = torch.zeros(self.exp.total, device=dev, dtype=torch.bfloat16)
            for s in exp:
                sl = slice(s.offset, s.offset + s.numel)
                self.exp_master[sl].copy_(s.param.detach().reshape(-1))
                self.exp_param[sl].copy_(self.exp_master[sl])
                s.param.data = self.exp_param[sl].view(s.param.shape)
            self.exp_grad = torch.zeros(self.exp.total, device=dev, dtype=torch.float32)
            self.exp_m = torch.zeros_like(self.exp_grad)
            self.exp_v = torch.zeros_like(self.exp_grad)
            for s in exp:
                s.param.main_grad = self.exp_grad[s.offset:s.offset + s.numel].view(s.param.shape)

        self.small_param = torch.zeros(self.small.total, device=dev, dtype=torch.float32)
        self.small_grad = torch.zeros(self.small.total, device=dev, dtype=torch.float32)
        self.small_m = torch.zeros_like(self.small_param)
        self.small_v = torch.zeros_like(self.small_param)
        for s in small:
            self.small_param[s.offset:s.offset + s.numel] = s.param.detach().float().reshape(-1).to(dev)
            s.param.data = self.small_param[s.offset:s.offset + s.numel].view(s.param.shape)
            s.param.main_grad = self.small_grad[s.offset:s.offset + s.numel].view(s.param.shape)
        for _, p in frozen:
            p.data = p.data.to(dev)
        for b in self.model.buffers():
            b.data = b.data.to(dev)
        self.small_wd = torch.ones(self.small.total, device=dev, dtype=torch.float32)
        for s in small:
            if not weight_decay_mask(s.name):
                self.small_wd[s.offset:s.offset + s.numel] = 0.0

    def _alloc_sharded_group(self, big: list, buckets: list, total_b: int) -> None:
        """Device storage of the sharded group: resident bf16 compute copy and fp32 gradient accumulator (full, flat),
        fp32 master / moments / reduced gradient (this rank's slices)."""
        dev = self.device
        # fp32 master values come from the model's initialisation.  Parameters are consumed one at a time (they may
        # already live on the device): the bf16 compute copy and this rank's slice of the fp32 master are filled
        # from a parameter, then its own storage is released by re-pointing it at the flat buffer.
        self.param_flat = self._alloc_symmetric(total_b, torch.bfloat16)
        self.param_flat.zero_()
        self.grad_flat = self._alloc_symmetric(total_b, torch.float32)
        self.grad_flat.zero_()
        self.master = torch.zeros(self.shard_size, device=dev, dtype=torch.float32)
        self.exp_avg = torch.zeros(self.shard_size, device=dev, dtype=torch.float32)
        self.exp_avg_sq = torch.zeros(self.shard_size, device=dev, dtype=torch.float32)
        self.grad_shard = torch.empty(self.shard_size, device=dev, dtype=torch.float32)
        # per-element weight decay is uniform over the big group (only the router bias is exempt and it is frozen)
        for s in big:
            src = s.param.detach().reshape(-1)
            self.param_flat[s.offset:s.offset + s.numel].copy_(src)
            for a, b, loc in self._overlaps(s.offset, s.offset + s.numel):
                self.master[loc:loc + (b - a)].copy_(src[a - s.offset:b - s.offset])
            del src
            s.param.data = self.param_flat[s.offset:s.offset + s.numel].view(s.param.shape)
            s.param.main_grad = self.grad_flat[s.offset:s.offset + s.numel].view(s.param.shape)
            s.bucket = self._bucket_index.get(bucket_of(s.name), 0) if len(buckets) > 1 else 0

    def _overlaps(self, lo: int, hi: int):
        """Parts of the flat range ``[lo, hi)`` that this rank's shard holds: ``(flat_a, flat_b, local offset)``."""
        for _, a, b, loc in self.segments:
            x, y = max(a, lo), min(b, hi)
            if x < y:
                yield x, y, loc + (x - a)

    def _gather_flat(self, local: torch.Tensor) -> torch.Tensor:
        """All ranks' shard arrays reassembled into the flat layout (bucket by bucket, rank slices in rank order)."""
        if self.world == 1:
            return local
        every = torch.empty(self.world, self.shard_size, device=self.device, dtype=local.dtype)
        dist.all_gather_into_tensor(every.view(-1), local.contiguous(), group=self.group)
        full = torch.empty(self.big.total, device=self.device, dtype=local.dtype)
        for (_, boff, blen), (_, _, _, loc) in zip(self.buckets, self.segments):
            sl = blen // self.world
            full[boff:boff + blen].view(self.world, sl).copy_(every[:, loc:loc + sl])
        return full

    def _matrix_aligned_layout(self, big: list) -> int:
        """Muon orthogonalises whole matrices, so under Muon no parameter may straddle two optimizer shards:
        parameters are packed greedily (largest first) into one bin per rank, a bin being that rank's contiguous
        shard of the flat buffers.  Returns the flat total (``world`` bins of the largest bin's size)."""
        loads = [0] * self.world
        placed: list[tuple[_Slot, int, int]] = []
        for s in sorted(big, key=lambda t: -t.numel):
            b = min(range(self.world), key=lambda i: loads[i])
            placed.append((s, b, loads[b]))
            loads[b] = _round_up(loads[b] + s.numel, _ALIGN)
        bin_size = _round_up(max(loads), 1024)
        for s, b, off in placed:
            s.offset = b * bin_size + off
        return bin_size * self.world

    def _alloc_symmetric(self, numel: int, dtype: torch.dtype) -> torch.Tensor:
        """Flat buffers live in symmetric (peer-mappable) memory when the peer-memory path may be used."""
        if self.world > 1 and bool(self.config.fused_collectives):
            try:
                import torch.distributed._symmetric_memory as symm

                return symm.empty(numel, dtype=dtype, device=self.device)
            except Exception:
                pass
        return torch.empty(numel, dtype=dtype, device=self.device)

    # ------------------------------------------------------------------ helpers
    def named_master_parameters(self) -> dict[str, torch.Tensor]:
        """Full fp32 master tensors by name (gathers the shards; used by checkpointing and tests)."""
        full = self._gather_flat(self.master)
        out = {s.name: full[s.offset:s.offset + s.numel].view(s.param.shape).clone() for s in self.big.slots}
        for s in self.small.slots:
            out[s.name] = s.param.detach().clone()
        for n, p in self.model.named_parameters():
            if n not in out:
                out[n] = p.detach().clone()
        return out

    def zero_grad(self, force: bool = False) -> None:
        """Clear the gradient accumulators.  The flat buffer of the sharded group is skipped when the previous
        step's bucket pulls have already cleared it (each owner zeroes what it has consumed, on every rank)."""
        if force or not self._flat_cleared_by_pull:
            self.grad_flat.zero_()
        self._flat_cleared_by_pull = False
        self.small_grad.zero_()
        if self.exp.slots:
            self.exp_grad.zero_()

    def _fold_autograd_grads(self, slots=None) -> None:
        """Parameters whose ops returned ordinary autograd gradients: add them into the flat buffers.  A gradient
        that arrives for a bucket whose reduction has already been issued marks the bucket for a second,
        accumulating pull."""
        groups = (slots,) if slots is not None else (self.big.slots, self.small.slots, self.exp.slots)
        for grp in groups:
            for s in grp:
                g = s.param.grad
                if g is not None:
                    s.param.main_grad.add_(g.to(torch.float32))
                    s.param.grad = None
                    if grp is self.big.slots and s.bucket in self._pulled:
                        self._late.add(s.bucket)

    # ------------------------------------------------------------------ step
    def backward(self, loss: torch.Tensor) -> None:
        loss.backward()
        self._fold_autograd_grads()

    def _micro_batch(self, micro: dict, last: bool):
        """Forward + backward of one micro-batch.  On the last one of a step (peer-memory path) every decoder layer
        reports when the backward pass has left it, and its bucket's reduce-scatter starts on the side stream right
        away; the hook has to be in place during the forward pass, which arms it on the layers' inputs."""
        from mintext_b200.models import transformer as tfm
        from mintext_b200.trainer import compute_loss

        overlap = last and self._overlap_ok()
        if overlap:
            tfm.set_backward_layer_hook(self._on_layer_backward_done)
        try:
            loss, aux = compute_loss(None, self.model, self.config, micro)
            self.backward(loss)
        finally:
            if overlap:
                tfm.set_backward_layer_hook(None)
        return aux

    def _overlap_ok(self) -> bool:
        if not (self.use_fused and len(self.buckets) > 1) or os.environ.get("MT_OVERLAP_GRAD_REDUCE", "1") == "0":
            return False
        if self._has_tp_replicated is None:
            self._has_tp_replicated = any(getattr(s.param, "tp_replicated_compute", False) for s in self.big.slots)
        return not self._has_tp_replicated  # those gradients are rescaled before the reduction

    def _on_layer_backward_done(self, layer: int) -> None:
        b = self._bucket_index.get(layer + 1)
        if b is None or b in self._pulled:
            return
        if self._slots_of_bucket is None:
            self._slots_of_bucket = {}
            for s in self.big.slots:
                self._slots_of_bucket.setdefault(s.bucket, []).append(s)
        for s in self._slots_of_bucket.get(b, ()):  # gradients that came back through autograd so far
            g = s.param.grad
            if g is not None:
                s.param.main_grad.add_(g.to(torch.float32))
                s.param.grad = None
        self._comm.pull_bucket_async(b)
        self._pulled.add(b)

    def _reduce_sharded_group(self) -> None:
        """``grad_shard`` <- this rank's slices of the gradients summed over all ranks."""
        W = self.world
        if self.use_fused and len(self.buckets) > 1:
            self._comm.finish_bucket_pulls(self._pulled, self._late)
            self._pulled, self._late = set(), set()
            self._flat_cleared_by_pull = True
        elif self.use_fused:
            self._comm.reduce_scatter_grads(self.grad_shard)
        else:
            for (_, boff, blen), (_, _, _, loc) in zip(self.buckets, self.segments):
                dist.reduce_scatter_tensor(self.grad_shard[loc:loc + blen // W], self.grad_flat[boff:boff + blen],
                                           group=self.group)

    def _update_sharded_group(self, gshard: torch.Tensor, lr: float, bc1: float, bc2: float, inv: float) -> None:
        """AdamW on this rank's slices and publication of the updated bf16 values to every rank (multi-rank runs)."""
        cfg = self.config
        e = ext()
        if self.use_fused:
            self._comm.adamw_and_publish(gshard, lr, bc1, bc2, inv, self._clip)
            return
        for (_, boff, blen), (_, a, b, loc) in zip(self.buckets, self.segments):
            sl = slice(loc, loc + (b - a))
            pslice = self.param_flat[a:b]
            e.adamw_step(self.master[sl], self.exp_avg[sl], self.exp_avg_sq[sl], gshard[sl], pslice, lr, cfg.adam_b1,
                         cfg.adam_b2, cfg.adam_eps, cfg.weight_decay, bc1, bc2, inv, self._clip)
            dist.all_gather_into_tensor(self.param_flat[boff:boff + blen], pslice, group=self.group)

    def optimizer_step(self, num_micro: int = 1) -> dict:
        """Reduce gradients, clip, update, re-publish bf16 weights.  Returns device scalars."""
        cfg = self.config
        e = ext()
        W = self.world
        inv = 1.0 / (num_micro * W)  # micro-batch losses are means over local tokens
        lr = float(self.schedule(self.step_count))
        self.step_count += 1
        t = self.step_count
        bc1 = 1.0 - cfg.adam_b1 ** t
        bc2 = 1.0 - cfg.adam_b2 ** t

        # sub-layers that every rank of a tensor-parallel group computes in full hold identical gradients there
        # (of the group's summed loss): divide by the group size so that the cross-rank sum counts them once
        from mintext_b200.parallel.tp import current_tp

        tp = current_tp()
        if tp is not None and tp.size > 1:
            for grp in (self.big, self.small):
                for s in grp.slots:
                    if getattr(s.param, "tp_replicated_compute", False):
                        s.param.main_grad.mul_(1.0 / tp.size)
        # 1. gradient reduction
        if W > 1:
            self._reduce_sharded_group()
            dist.all_reduce(self.small_grad, group=self.group)
            gshard = self.grad_shard
        else:
            gshard = self.grad_flat
        # 2. global norm of the averaged gradient
        if W > 1 and self.use_fused and len(self.buckets) == 1:
            self._sumsq.copy_(self._sumsq_shard)  # produced by the pull-reduce kernel
        else:
            self._sumsq.zero_()
            e.sumsq(gshard, self._sumsq)
        if self.exp.slots:
            # slices are disjoint across ranks up to their replicas: sum over the replicas, count each slice once
            for lo, hi, grp, size in self._exp_ranges():
                seg = self.exp_grad[lo:hi]
                if grp is not None:
                    dist.all_reduce(seg, group=grp)
                tmp = torch.zeros_like(self._sumsq)
                e.sumsq(seg, tmp)
                self._sumsq.add_(tmp / size)
        if W > 1:
            dist.all_reduce(self._sumsq, group=self.group)
        e.sumsq(self.small_grad, self._sumsq)
        grad_norm = torch.sqrt(self._sumsq) * inv
        if cfg.gradient_clip_threshold > 0:
            thr = float(cfg.gradient_clip_threshold)
            torch.div(thr, torch.clamp(grad_norm, min=thr), out=self._clip)
        else:
            self._clip.fill_(1.0)
        # 3. fused AdamW on the shard (+ 4. publication of the bf16 copy)
        if self.use_muon:
            lo = self.rank * self.shard_size
            pshard = self.param_flat[lo:lo + self.shard_size]
            self._muon_group(self.big.slots, lo, lo + self.shard_size, self.master, self.exp_avg, self.exp_avg_sq,
                             gshard, pshard, lr, bc1, bc2, inv, t)
            if W > 1 and self._muon_comm is not None:
                self._muon_comm.publish()
            elif W > 1:
                dist.all_gather_into_tensor(self.param_flat, pshard, group=self.group)
        elif W > 1:
            self._update_sharded_group(gshard, lr, bc1, bc2, inv)
        else:
            e.adamw_step(self.master, self.exp_avg, self.exp_avg_sq, gshard, self.param_flat, lr, cfg.adam_b1,
                         cfg.adam_b2, cfg.adam_eps, cfg.weight_decay, bc1, bc2, inv, self._clip)
        if self.exp.slots and self.use_muon:
            self._muon_group(self.exp.slots, 0, self.exp.total, self.exp_master, self.exp_m, self.exp_v, self.exp_grad,
                             self.exp_param, lr, bc1, bc2, inv, t)
        elif self.exp.slots:
            e.adamw_step(self.exp_master, self.exp_m, self.exp_v, self.exp_grad, self.exp_param, lr, cfg.adam_b1,
                         cfg.adam_b2, cfg.adam_eps, cfg.weight_decay, bc1, bc2, inv, self._clip)
        self._small_adamw(lr, bc1, bc2, inv)
        self.kernel_launches += 4
        from mintext_b200.ops import functional as F

        F.bump_weight_version()  # quantised weight copies kept by the layers are stale now
        return {"grad_norm": grad_norm, "learning_rate": lr}

    def _muon_group(self, slots, lo, hi, master, mom, second, grad, param_out, lr, bc1, bc2, inv, t) -> None:
        """Muon for the matrices, AdamW for everything else, over the slots held in ``[lo, hi)`` of a flat group
        (mintext/optim/optimizer.py:117-168: Nesterov momentum with optax's bias correction, Newton-Schulz,
        shape-dependent scale, decoupled weight decay)."""
        from mintext_b200.ops import muon as muon_ops
        from mintext_b200.optim.optimizer import (muon_matrix_view, muon_shape_scale, muon_slice_axis,
                                                  muon_sliced_update)
        from mintext_b200.parallel.tp import current_tp

        cfg = self.config
        e = ext()
        beta = cfg.muon_beta
        tp = current_tp()
        tp_group = tp.group if (tp is not None and tp.size > 1) else None
        for s in slots:
            if s.offset < lo or s.offset + s.numel > hi:
                continue
            a = s.offset - lo
            view = muon_matrix_view(s.name, tuple(s.param.shape))
            if view is None:
                n = min(_round_up(s.numel, _ALIGN), hi - s.offset)  # the padding behind a slot has zero gradients
                sl = slice(a, a + n)
                e.adamw_step(master[sl], mom[sl], second[sl], grad[sl], param_out[sl], lr, cfg.adam_b1, cfg.adam_b2,
                             cfg.adam_eps, cfg.weight_decay if weight_decay_mask(s.name) else 0.0, bc1, bc2, inv,
                             self._clip)
                continue
            sl = slice(a, a + s.numel)
            b, r, c = view
            g = grad[sl] * (inv * self._clip)
            mu = mom[sl]
            mu.mul_(beta).add_(g, alpha=1 - beta)
            mu_hat = mu * (beta / (1 - beta ** (t + 1))) + g * ((1 - beta) / (1 - beta ** t))
            axis = muon_slice_axis(s.name, s.param) if tp_group is not None else None
            if axis is not None:
                # a tensor-parallel slice (rank-local group: every rank of the group walks the same slots in the same
                # order): Gram matrices summed over the group, shape factor of the whole matrix
                upd, scale = muon_sliced_update(mu_hat, view, axis, tp_group, cfg.muon_newton_schulz_steps,
                                                cfg.adam_eps, cfg.muon_consistent_rms)
                upd = upd.reshape(-1)
            else:
                upd = muon_ops.newton_schulz(mu_hat.view(b, r, c), cfg.muon_newton_schulz_steps,
                                             cfg.adam_eps).reshape(-1)
                scale = muon_shape_scale(r, c, cfg.muon_consistent_rms)
            wd = cfg.weight_decay if weight_decay_mask(s.name) else 0.0
            w = master[sl]
            w.add_(upd * scale + wd * w, alpha=-lr)
            param_out[sl].copy_(w)

    def _small_adamw(self, lr, bc1, bc2, inv) -> None:
        cfg = self.config
        g = self.small_grad * (inv * self._clip)
        self.small_m.mul_(cfg.adam_b1).add_(g, alpha=1 - cfg.adam_b1)
        self.small_v.mul_(cfg.adam_b2).addcmul_(g, g, value=1 - cfg.adam_b2)
        upd = (self.small_m / bc1) / ((self.small_v / bc2).sqrt() + cfg.adam_eps)
        self.small_param.add_(upd + cfg.weight_decay * self.small_wd * self.small_param, alpha=-lr)

    def _exp_ranges(self):
        """Ranges of the rank-local (tensor- / expert-parallel) flat buffers with the group that holds replicas of
        them and its size: one range normally, two when tensor and expert parallelism are combined."""
        total = self.exp.total
        if self._exp_split is None:
            return [(0, total, self.local_reduce_group, self.local_reduce_size)]
        out = []
        if self._exp_split > 0:
            out.append((0, self._exp_split, self.local_reduce_group, self.local_reduce_size))
        if self._exp_split < total:
            out.append((self._exp_split, total, self.expert_reduce_group, self.expert_reduce_size))
        return out

    def param_norm(self) -> torch.Tensor:
        s = torch.zeros(1, device=self.device, dtype=torch.float32)
        ext().sumsq(self.master, s)
        for lo, hi, _, size in (self._exp_ranges() if self.exp.slots else ()):
            tmp = torch.zeros_like(s)
            ext().sumsq(self.exp_master[lo:hi], tmp)
            s.add_(tmp / size)
        if self.world > 1:
            dist.all_reduce(s, group=self.group)
        ext().sumsq(self.small_param, s)
        return torch.sqrt(s)

    def train_step(self, batch: dict, num_micro: int | None = None) -> dict:
        """``batch`` holds this rank's rows (``[B_local, S]`` token tensors on the device).  Runs ``num_micro``
        micro-batches (default ``gradient_accumulation_steps``), then one optimizer step."""
        from mintext_b200.trainer import compute_loss

        cfg = self.config
        n = num_micro or int(cfg.gradient_accumulation_steps)
        B = batch["input_tokens"].shape[0]
        mb = B // n
        self.zero_grad()
        loss_sum = torch.zeros((), device=self.device, dtype=torch.float32)
        counts = None
        for i in range(n):
            micro = {k: v[i * mb:(i + 1) * mb] for k, v in batch.items()}
            aux = self._micro_batch(micro, last=(i == n - 1))
            loss_sum += aux["loss"].float()
            if aux.get("moe_expert_counts") is not None:
                counts = aux["moe_expert_counts"] if counts is None else counts + aux["moe_expert_counts"]
        pnorm = self.param_norm()
        loss_mean = loss_sum / n
        if self.world > 1:
            dist.all_reduce(loss_mean, group=self.group)
            loss_mean /= self.world
            if counts is not None:
                dist.all_reduce(counts, group=self.group)
        if cfg.nan_policy != "ignore":
            from mintext_b200.parallel.health import apply_nan_policy

            # the all-reduced loss is the same on every rank, so all ranks take the same decision
            if apply_nan_policy(cfg.nan_policy, float(loss_mean), self.step_count):
                self._abandon_step()
                return {"loss": loss_mean, "param_norm": pnorm, "moe_expert_counts": None, "z_loss": aux["z_loss"],
                        "grad_norm": torch.full((), float("nan"), device=self.device),
                        "learning_rate": float(self.schedule(self.step_count)), "skipped": True}
        with nvtx_range("optimizer_step"):
            out = self.optimizer_step(n)
        out.update({"loss": loss_mean, "param_norm": pnorm, "moe_expert_counts": counts, "z_loss": aux["z_loss"]})
        return out

    def _abandon_step(self) -> None:
        """Drop the gradients of a skipped step.  Bucket reductions that were already issued are left to finish (every
        rank takes the same decision), then everything is cleared."""
        if self._comm is not None and self._pulled:
            self._comm.wait_side_stream()
            self._comm.barrier()  # no peer is still pulling from (or clearing) this rank's buffer
        self._pulled, self._late = set(), set()
        self.zero_grad(force=True)

    def check(self) -> None:
        """Raise if any kernel recorded a bounded-wait expiry since the last check (synchronises)."""
        check_status(self.device)

    # ------------------------------------------------------------------ evaluation / MoE bias / checkpoints
    @torch.no_grad()
    def eval_step(self, batch: dict) -> dict:
        from mintext_b200.trainer import compute_loss

        loss, _ = compute_loss(None, self.model, self.config, batch)
        loss = loss.detach().float()
        if self.world > 1:
            dist.all_reduce(loss, group=self.group)
            loss /= self.world
        return {"eval_loss": loss}

    @torch.no_grad()
    def update_expert_biases(self, expert_counts: torch.Tensor | None) -> None:
        """``bias += rate * sign(mean_count - count)`` per MoE layer, counts taken over the global batch."""
        if expert_counts is None:
            return
        rate = self.config.e_score_correction_bias_update_rate
        names = sorted((n for n, _ in self.model.named_parameters() if n.endswith("e_score_correction_bias")),
                       key=lambda n: int(n.split(".")[1]))
        params = dict(self.model.named_parameters())
        for name, counts in zip(names, expert_counts):
            c = counts.float()
            params[name].add_(rate * torch.sign(c.mean() - c))

    params_only_restore = False

    def checkpoint_tree(self) -> dict:
        """Flat fp32 master / moment buffers are saved as one chunk per rank (``flat_range`` = the rank's slice
        of the flat layout); small replicated and frozen parameters are saved by name from rank 0."""
        def chunks(local: torch.Tensor) -> list[dict]:
            # one chunk per bucket slice this rank holds: (flat range, the matching part of the shard array)
            return [{"tensor": local[loc:loc + (b - a)], "writer_rank": self.rank, "flat_range": (a, b),
                     "flat_total": self.big.total, "suffix": f".{a}-{b}"} for _, a, b, loc in self.segments]

        tree: dict = {
            "step": self.step_count,
            "layout/big": {"tensor": json.dumps([[s.name, s.offset, s.numel, list(s.param.shape)] for s in self.big.slots])},
            "opt_state/flat_master": chunks(self.master),
            "opt_state/flat_exp_avg": chunks(self.exp_avg),
            "opt_state/flat_exp_avg_sq": chunks(self.exp_avg_sq),
        }
        # expert- / tensor-parallel parameters: this rank's slice along the parameter's shard dimension; of the
        # data-parallel replicas that hold the same slice only the first writes it
        def first_replica(slot) -> bool:
            grp = self.local_reduce_group
            if self._exp_split is not None and slot.offset >= self._exp_split:
                grp = self.expert_reduce_group
            return grp is None or dist.get_rank(grp) == 0

        for s in self.exp.slots:
            dim, idx, cnt = getattr(s.param, "shard_spec", (0, self.rank, self.world))
            meta = {"writer_rank": self.rank if first_replica(s) else -1, "shard": (int(dim), int(idx), int(cnt)),
                    "suffix": f".shard{idx}of{cnt}"}
            sl = slice(s.offset, s.offset + s.numel)
            tree[f"params/{s.name}"] = {"tensor": self.exp_master[sl].view(s.param.shape), **meta}
            tree[f"opt_state/mu/{s.name}"] = {"tensor": self.exp_m[sl].view(s.param.shape), **meta}
            tree[f"opt_state/nu/{s.name}"] = {"tensor": self.exp_v[sl].view(s.param.shape), **meta}
        for s in self.small.slots:
            tree[f"params/{s.name}"] = s.param.detach()
            tree[f"opt_state/mu/{s.name}"] = self.small_m[s.offset:s.offset + s.numel].view(s.param.shape)
            tree[f"opt_state/nu/{s.name}"] = self.small_v[s.offset:s.offset + s.numel].view(s.param.shape)
        for n, p in self.model.named_parameters():
            if not p.requires_grad:
                tree[f"params/{n}"] = p.detach()
        return tree

    @torch.no_grad()
    def load_checkpoint_tree(self, read) -> None:
        paths = set(getattr(read, "paths", []))
        if "opt_state/flat_master" in paths:
            saved = {row[0]: row for row in json.loads(read("layout/big"))}
            mine = {s.name: s for s in self.big.slots}
            for n, s in mine.items():
                if n not in saved or saved[n][2] != s.numel:
                    raise ValueError(f"checkpoint has no parameter '{n}' of {s.numel} elements")
            same = all(saved[n][1] == s.offset for n, s in mine.items())
            kinds = [("opt_state/flat_master", self.master)]
            if not self.params_only_restore:
                kinds += [("opt_state/flat_exp_avg", self.exp_avg), ("opt_state/flat_exp_avg_sq", self.exp_avg_sq)]
            if same:
                for path, dst in kinds:
                    for _, a, b, loc in self.segments:
                        dst[loc:loc + (b - a)].copy_(read(path, (a, b)))
            else:
                # the flat layout depends on the optimizer and the rank count (bucket lengths are rounded to the
                # rank count; Muon packs whole matrices per rank): look every parameter up by name in the saved
                # layout and copy the parts this rank holds
                for s in self.big.slots:
                    so = saved[s.name][1]
                    for a, b, loc in self._overlaps(s.offset, s.offset + s.numel):
                        for path, dst in kinds:
                            dst[loc:loc + (b - a)] = read(path, (so + a - s.offset, so + b - s.offset)).to(self.device)
        else:  # a per-name checkpoint written by the CPU trainer
            for s in self.big.slots:
                full = read(f"params/{s.name}").float().reshape(-1)
                for a, b, loc in self._overlaps(s.offset, s.offset + s.numel):
                    self.master[loc:loc + (b - a)] = full[a - s.offset:b - s.offset].to(self.device)
        for s in self.exp.slots:
            spec = tuple(getattr(s.param, "shard_spec", (0, self.rank, self.world)))
            sl = slice(s.offset, s.offset + s.numel)
            self.exp_master[sl] = read(f"params/{s.name}", shard=spec).reshape(-1).float().to(self.device)
            if not self.params_only_restore and f"opt_state/mu/{s.name}" in paths:
                self.exp_m[sl] = read(f"opt_state/mu/{s.name}", shard=spec).reshape(-1).to(self.device)
                self.exp_v[sl] = read(f"opt_state/nu/{s.name}", shard=spec).reshape(-1).to(self.device)
        if self.exp.slots:
            self.exp_param.copy_(self.exp_master.to(torch.bfloat16))
        for s in self.small.slots:
            s.param.copy_(read(f"params/{s.name}").to(self.device))
            if not self.params_only_restore and f"opt_state/mu/{s.name}" in paths:
                self.small_m[s.offset:s.offset + s.numel] = read(f"opt_state/mu/{s.name}").reshape(-1).to(self.device)
                self.small_v[s.offset:s.offset + s.numel] = read(f"opt_state/nu/{s.name}").reshape(-1).to(self.device)
        for n, p in self.model.named_parameters():
            if not p.requires_grad and f"params/{n}" in paths:
                p.copy_(read(f"params/{n}").to(self.device))
        if not self.params_only_restore:
            self.step_count = int(read("step"))
        self._publish_master()

    def _publish_master(self) -> None:
        """Rebuild the resident bf16 compute copy from the fp32 master shards."""
        from mintext_b200.ops import functional as F

        F.bump_weight_version()
        for (_, boff, blen), (_, a, b, loc) in zip(self.buckets, self.segments):
            mine = self.master[loc:loc + (b - a)].to(torch.bfloat16)
            if self.world > 1:
                dist.all_gather_into_tensor(self.param_flat[boff:boff + blen], mine, group=self.group)
            else:
                self.param_flat[a:b].copy_(mine)

    def reset_step(self) -> None:
        self.step_count = 0
        self.exp_avg.zero_()
        self.exp_avg_sq.zero_()
        self.small_m.zero_()
        self.small_v.zero_()

    @torch.no_grad()
    def refresh_from_model(self) -> None:
        """Parameters were overwritten in place (e.g. by an HF import into the bf16 views): re-derive the master
        shards from them."""
        from mintext_b200.ops import functional as F

        F.bump_weight_version()
        for _, a, b, loc in self.segments:
            self.master[loc:loc + (b - a)].copy_(self.param_flat[a:b].float())


def local_batch_rows(global_batch: int, world: int, rank: int) -> tuple[int, int]:
    """Row range of the global batch that ``rank`` of ``world`` data-parallel ranks processes."""
    if global_batch % world != 0:
        raise ValueError(f"global batch {global_batch} is not divisible by {world} ranks")
    per = global_batch // world
    return rank * per, (rank + 1) * per
