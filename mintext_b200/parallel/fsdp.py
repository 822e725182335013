"""Parameter-sharded engine mode (``fsdp_shard_params``): ZeRO-3 style storage on top of :class:`TrainEngine`.

The reference shards every weight over the ``fsdp`` axis (mintext/config.py:82, mintext/distributed/sharding.py:130-165)
and lets XLA insert the all-gathers and reduce-scatters.  The resident mode of the engine keeps the whole bf16 copy and
a whole fp32 gradient accumulator on every GPU (6 bytes per parameter before any optimizer state); this mode keeps, per
decoder layer, only the rank's ``1/N`` slice of both:

* **Weights.**  ``param_shard`` (bf16, ``1/N`` of every bucket, symmetric memory) is what persists.  A decoder layer
  computes from one of two staging slots (layer ``L`` uses slot ``L % 2``): before the layer runs, ``peer_gather``
  (csrc/comm/rs_optim.cu) copies slice ``r`` from rank ``r``'s shard buffer over NVLink on a side stream.  The gather of
  layer ``L + 1`` is issued when layer ``L`` starts (forward) and that of layer ``L - 2`` when the backward pass has
  left layer ``L`` (backward), so the consuming GEMMs find their weights in place.  Autograd's saved weight tensors
  are views of the slot, and the layer is always gathered into the same slot again before its backward runs.
* **Gradients.**  Weight-gradient epilogues add into a two-slot fp32 staging buffer (symmetric memory).  When the
  backward pass has left layer ``L`` its slot is reduce-scattered by ``grad_pull_bucket`` (every rank sums its slice
  from all peers and accumulates it into its persistent ``grad_shard``), followed by a barrier (every peer has read
  this rank's slot) and a local clearing of the slot, after which the layer two below may write it.  With gradient
  accumulation every micro-batch reduces every layer.
* **Bucket 0** (embedding, output head, final norm: used at both ends of the step) stays resident and follows the
  resident mode's path.

The optimizer step updates ``param_shard`` in place (no publication of layer weights); the next step's gathers read it.
"""

from __future__ import annotations

import os

import torch
import torch.distributed as dist

from mintext_b200.ops._ext import ext, status_word
from mintext_b200.parallel.engine import TrainEngine, bucket_of


class _ShardedComm:
    """Symmetric buffers, flags and streams of the parameter-sharded mode."""

    def __init__(self, engine: "ParamShardedEngine"):
        import torch.distributed._symmetric_memory as symm

        self.engine = engine
        group = engine.group or dist.group.WORLD
        self.rank, self.world = engine.rank, engine.world
        if self.world > 8:
            raise RuntimeError("the peer-memory path covers a single NVSwitch domain of at most 8 GPUs")
        dev = engine.device

        def ptrs(t):
            h = symm.rendezvous(t, group)
            self._handles.append(h)
            return [int(p) for p in h.buffer_ptrs]

        self._handles: list = []
        self.flags = symm.empty(64, dtype=torch.int32, device=dev).zero_()          # step-end barrier (compute stream)
        self.flags_side = symm.empty(64, dtype=torch.int32, device=dev).zero_()     # slot-release barrier (side stream)
        self.bucket_slots = int(ext().bucket_flag_slots())
        if len(engine.buckets) > self.bucket_slots:
            raise RuntimeError(f"{len(engine.buckets)} gradient buckets exceed the {self.bucket_slots} flag slots")
        self.bucket_flags = symm.empty(self.world * self.bucket_slots, dtype=torch.int32, device=dev).zero_()
        self.flag_ptrs = ptrs(self.flags)
        self.flag_side_ptrs = ptrs(self.flags_side)
        self.bflag_ptrs = ptrs(self.bucket_flags)
        self.shard_ptrs = ptrs(engine.param_shard)
        self.stage_grad_ptrs = ptrs(engine.stage_grad)
        self.res_grad_ptrs = ptrs(engine.res_grad) if engine.res_grad is not None else None
        self.res_param_ptrs = ptrs(engine.res_param) if engine.res_param is not None else None
        self.seq = 0
        self.seq_side = 0
        self.side = torch.cuda.Stream(device=dev)      # gradient reduce-scatters
        self.gather = torch.cuda.Stream(device=dev)    # weight gathers
        self.gather_blocks = int(os.environ.get("MT_PARAM_GATHER_BLOCKS", "32"))
        self.pull_blocks = int(os.environ.get("MT_GRAD_PULL_BLOCKS", "32"))
        # The per-layer reduce-scatter runs on the compute stream, between two layers' backward passes.  Running it
        # on the side stream under the next layer's backward (MT_FSDP_OVERLAP_REDUCE=1) is wired but off: on some
        # 2-GPU boxes it produced intermittently different updates whose cause has not been found.
        self.overlap_reduce = os.environ.get("MT_FSDP_OVERLAP_REDUCE", "0") == "1"
        torch.cuda.synchronize(dev)
        dist.barrier(group=group)

    def barrier(self) -> None:
        self.seq += 1
        ext().symm_barrier(self.flag_ptrs, self.rank, self.seq, status_word(self.engine.device))

    def barrier_side(self) -> None:
        self.seq_side += 1
        ext().symm_barrier(self.flag_side_ptrs, self.rank, self.seq_side, status_word(self.engine.device))


class ParamShardedEngine(TrainEngine):
    """:class:`TrainEngine` with layer weights and layer gradients sharded ``1/N`` (see the module docstring)."""

    sharded_params = True

    def __init__(self, model, config, device="cuda", group=None, local_reduce_group=None, expert_reduce_group=None):
        if not (dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1):
            raise ValueError("fsdp_shard_params needs more than one rank")
        if config.optimizer != "adamw" or not bool(config.fused_collectives) or config.torch_dtype != torch.bfloat16:
            raise ValueError("fsdp_shard_params runs on the peer-memory AdamW path in bf16 (optimizer=adamw, "
                             "fused_collectives=true, dtype=bfloat16)")
        from mintext_b200.parallel.tp import current_tp

        if current_tp() is not None and current_tp().size > 1:
            raise ValueError("fsdp_shard_params is not combined with tensor parallelism")
        super().__init__(model, config, device=device, group=group, local_reduce_group=local_reduce_group,
                         expert_reduce_group=expert_reduce_group)
        from mintext_b200.models import transformer as tfm

        self._sc = _ShardedComm(self)
        self._slot_layer: list[int | None] = [None, None]   # layer whose weights each staging slot holds (or will)
        self._slot_event: list = [None, None]               # completion of that gather
        self._slot_waited = [True, True]                    # the compute stream already waits for it
        self._grad_event: list = [None, None]               # completion of the last reduce-scatter of a gradient slot
        self._micro_index = 0
        self._round = 0
        self.num_layers = len(self._layer_bucket)
        tfm.set_forward_layer_hook(self._before_layer_forward)
        tfm.set_backward_layer_hook(self._after_layer_backward)

    # ------------------------------------------------------------------ storage
    def _use_symmetric_optimizer_comm(self) -> bool:
        return False

    def _alloc_sharded_group(self, big: list, buckets: list, total_b: int) -> None:
        dev = self.device
        if len(buckets) < 2:
            raise ValueError("fsdp_shard_params needs per-layer buckets (a decoder with at least one layer)")
        self.param_flat = None
        self.grad_flat = None
        self._layer_bucket: dict[int, int] = {}   # layer -> index into self.buckets
        self._res_index = None
        for i, (bid, _, _) in enumerate(buckets):
            if bid == 0:
                self._res_index = i
            else:
                self._layer_bucket[bid - 1] = i
        self.stage_len = max(blen for bid, _, blen in buckets if bid != 0)
        self.param_shard = self._alloc_symmetric(self.shard_size, torch.bfloat16)
        self.stage_param = torch.zeros(2 * self.stage_len, device=dev, dtype=torch.bfloat16)
        self.stage_grad = self._alloc_symmetric(2 * self.stage_len, torch.float32)
        self.stage_grad.zero_()
        self.res_param = self.res_grad = None
        if self._res_index is not None:
            rlen = buckets[self._res_index][2]
            self.res_param = self._alloc_symmetric(rlen, torch.bfloat16)
            self.res_param.zero_()
            self.res_grad = self._alloc_symmetric(rlen, torch.float32)
            self.res_grad.zero_()
        self.master = torch.zeros(self.shard_size, device=dev, dtype=torch.float32)
        self.exp_avg = torch.zeros(self.shard_size, device=dev, dtype=torch.float32)
        self.exp_avg_sq = torch.zeros(self.shard_size, device=dev, dtype=torch.float32)
        self.grad_shard = torch.zeros(self.shard_size, device=dev, dtype=torch.float32)
        start = {i: boff for i, (_, boff, _) in enumerate(buckets)}
        for s in big:
            src = s.param.detach().reshape(-1)
            for a, b, loc in self._overlaps(s.offset, s.offset + s.numel):
                self.master[loc:loc + (b - a)].copy_(src[a - s.offset:b - s.offset])
            s.bucket = self._bucket_index.get(bucket_of(s.name), 0)
            rel = s.offset - start[s.bucket]
            if s.bucket == self._res_index:
                self.res_param[rel:rel + s.numel].copy_(src)
                pview, gview = self.res_param[rel:rel + s.numel], self.res_grad[rel:rel + s.numel]
            else:
                layer = buckets[s.bucket][0] - 1
                base = (layer % 2) * self.stage_len + rel
                pview, gview = self.stage_param[base:base + s.numel], self.stage_grad[base:base + s.numel]
            del src
            s.param.data = pview.view(s.param.shape)
            s.param.main_grad = gview.view(s.param.shape)
        self.param_shard.copy_(self.master)  # fp32 -> bf16

    def _alloc_symmetric(self, numel: int, dtype: torch.dtype) -> torch.Tensor:
        import torch.distributed._symmetric_memory as symm

        return symm.empty(numel, dtype=dtype, device=self.device)

    # ------------------------------------------------------------------ weight gathers
    def _issue_gather(self, layer: int) -> None:
        """Queue the gather of ``layer`` into its slot behind everything the compute stream has been given so far
        (the slot's previous occupant is two layers away and no longer running by then)."""
        slot = layer % 2
        if self._slot_layer[slot] == layer:
            return
        sc = self._sc
        cur = torch.cuda.current_stream(self.device)
        free = torch.cuda.Event()
        free.record(cur)
        sc.gather.wait_event(free)
        bidx = self._layer_bucket[layer]
        _, _, blen = self.buckets[bidx]
        _, _, _, loc = self.segments[bidx]
        sl = blen // self.world
        dst = self.stage_param[slot * self.stage_len:slot * self.stage_len + blen]
        with torch.cuda.stream(sc.gather):
            ext().peer_gather(sc.shard_ptrs, loc, 0, sl, dst, sc.gather_blocks)
            done = torch.cuda.Event()
            done.record(sc.gather)
        self._slot_layer[slot] = layer
        self._slot_event[slot] = done
        self._slot_waited[slot] = False
        self.kernel_launches += 1

    def _wait_gather(self, layer: int) -> None:
        slot = layer % 2
        if self._slot_layer[slot] != layer:
            self._issue_gather(layer)
        if not self._slot_waited[slot]:
            torch.cuda.current_stream(self.device).wait_event(self._slot_event[slot])
            self._slot_waited[slot] = True

    def _before_layer_forward(self, layer: int) -> None:
        self._wait_gather(layer)
        if layer + 1 < self.num_layers:
            self._issue_gather(layer + 1)

    def _after_layer_backward(self, layer: int) -> None:
        """The backward pass has left ``layer``: reduce its gradient slot, make sure the next layer down has its
        weights and its gradient slot is free, and prefetch the layer after that."""
        sc = self._sc
        cur = torch.cuda.current_stream(self.device)
        bidx = self._layer_bucket.get(layer)
        if bidx is None:
            return
        slot = layer % 2
        for s in self._slots_by_bucket().get(bidx, ()):  # gradients that came back through autograd
            g = s.param.grad
            if g is not None:
                s.param.main_grad.add_(g.to(torch.float32))
                s.param.grad = None
        sc.side.wait_stream(cur)
        _, _, blen = self.buckets[bidx]
        _, _, _, loc = self.segments[bidx]
        sl = blen // self.world
        with torch.cuda.stream(sc.side if sc.overlap_reduce else cur):
            # the slot is written again two layers later: no remote clearing stores (their arrival at the peer is not
            # ordered with the barrier that follows); every rank clears its own slot once all peers have read it
            ext().grad_pull_bucket(sc.stage_grad_ptrs, sc.bflag_ptrs, self.rank, bidx, self._pull_seq(),
                                   slot * self.stage_len + self.rank * sl, self.grad_shard[loc:loc + sl],
                                   self._micro_index > 0, False, True,
                                   max(sc.pull_blocks, min(296, sl * 4 // (2 << 20))) if sc.overlap_reduce else 0,
                                   status_word(self.device))
            sc.barrier_side()  # every rank has pulled its slice of this slot
            self.stage_grad[slot * self.stage_len:slot * self.stage_len + blen].zero_()
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream(self.device))
        self._grad_event[slot] = ev
        self._pulled.add(bidx)
        self.kernel_launches += 2
        if layer >= 1:
            other = (layer - 1) % 2
            if self._grad_event[other] is not None:  # the slot layer - 1 writes was last reduced for layer + 1
                cur.wait_event(self._grad_event[other])
            self._wait_gather(layer - 1)
        if layer >= 2:
            self._issue_gather(layer - 2)

    def _pull_seq(self) -> int:
        return self._round  # one per micro-batch, the same on every rank

    def _slots_by_bucket(self) -> dict:
        if self._slots_of_bucket is None:
            self._slots_of_bucket = {}
            for s in self.big.slots:
                self._slots_of_bucket.setdefault(s.bucket, []).append(s)
        return self._slots_of_bucket

    # ------------------------------------------------------------------ step
    def zero_grad(self, force: bool = False) -> None:
        if self.res_grad is not None and (force or not self._flat_cleared_by_pull):
            self.res_grad.zero_()
        if force:
            self.stage_grad.zero_()
        self._flat_cleared_by_pull = False
        self.small_grad.zero_()
        if self.exp.slots:
            self.exp_grad.zero_()
        self._micro_index = 0

    def _fold_autograd_grads(self, slots=None) -> None:
        groups = (slots,) if slots is not None else (self.big.slots, self.small.slots, self.exp.slots)
        for grp in groups:
            for s in grp:
                g = s.param.grad
                if g is None:
                    continue
                if grp is self.big.slots and s.bucket != self._res_index:
                    raise RuntimeError(f"gradient of '{s.name}' arrived after its layer's gradient slot was reduced; "
                                       "fsdp_shard_params cannot accumulate it")
                s.param.main_grad.add_(g.to(torch.float32))
                s.param.grad = None

    def _micro_batch(self, micro: dict, last: bool):
        from mintext_b200.trainer import compute_loss

        self._round += 1
        cur = torch.cuda.current_stream(self.device)
        cur.wait_stream(self._sc.side)  # gradient slots of the previous micro-batch are reduced and released
        self._grad_event = [None, None]
        loss, aux = compute_loss(None, self.model, self.config, micro)
        self.backward(loss)
        self._micro_index += 1
        return aux

    def _overlap_ok(self) -> bool:
        return False

    def _reduce_sharded_group(self) -> None:
        sc = self._sc
        cur = torch.cuda.current_stream(self.device)
        cur.wait_stream(sc.side)
        missing = [l for l, b in self._layer_bucket.items() if b not in self._pulled]
        if missing:
            raise RuntimeError(f"layers {missing} never reported the end of their backward pass")
        if self._res_index is not None:
            self._round += 1
            _, _, blen = self.buckets[self._res_index]
            _, _, _, loc = self.segments[self._res_index]
            sl = blen // self.world
            ext().grad_pull_bucket(sc.res_grad_ptrs, sc.bflag_ptrs, self.rank, self._res_index, self._round,
                                   self.rank * sl, self.grad_shard[loc:loc + sl], False, True, True, 0,
                                   status_word(self.device))
            self._flat_cleared_by_pull = True
        self._pulled, self._late = set(), set()

    def _update_sharded_group(self, gshard: torch.Tensor, lr: float, bc1: float, bc2: float, inv: float) -> None:
        cfg = self.config
        e = ext()
        sc = self._sc
        for i, (_, a, b, loc) in enumerate(self.segments):
            sl = slice(loc, loc + (b - a))
            if i == self._res_index:
                e.adamw_publish(self.master[sl], self.exp_avg[sl], self.exp_avg_sq[sl], gshard[sl], sc.res_param_ptrs,
                                a - self.buckets[i][1], lr, cfg.adam_b1, cfg.adam_b2, cfg.adam_eps, cfg.weight_decay, bc1,
                                bc2, inv, self._clip)
            else:
                e.adamw_step(self.master[sl], self.exp_avg[sl], self.exp_avg_sq[sl], gshard[sl], self.param_shard[sl], lr,
                             cfg.adam_b1, cfg.adam_b2, cfg.adam_eps, cfg.weight_decay, bc1, bc2, inv, self._clip)
        sc.barrier()  # every rank's shard is final (and the resident bucket published) before anyone gathers again
        self._invalidate_slots()
        for layer in range(min(2, self.num_layers)):  # the next step's first layers, under the rest of this step
            self._issue_gather(layer)

    def _invalidate_slots(self) -> None:
        self._slot_layer = [None, None]
        self._slot_waited = [True, True]

    def _abandon_step(self) -> None:
        cur = torch.cuda.current_stream(self.device)
        cur.wait_stream(self._sc.side)
        self._sc.barrier()
        self._pulled, self._late = set(), set()
        self.zero_grad(force=True)

    # ------------------------------------------------------------------ whole-tensor access
    def _publish_master(self) -> None:
        from mintext_b200.ops import functional as F

        F.bump_weight_version()
        self.param_shard.copy_(self.master)
        if self._res_index is not None:
            _, a, b, loc = self.segments[self._res_index]
            boff, blen = self.buckets[self._res_index][1:]
            mine = self.master[loc:loc + (b - a)].to(torch.bfloat16)
            dist.all_gather_into_tensor(self.res_param[:blen], mine, group=self.group)
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        self._invalidate_slots()

    def refresh_from_model(self) -> None:
        raise NotImplementedError("with fsdp_shard_params the layer weights are not resident: import weights through "
                                  "a checkpoint (load_checkpoint_tree) instead of writing into the model's tensors")

    def close(self) -> None:
        """Detach the layer hooks (they are process-wide)."""
        from mintext_b200.models import transformer as tfm

        tfm.set_forward_layer_hook(None)
        tfm.set_backward_layer_hook(None)

    def gather_layer_weights(self, layer: int) -> None:
        """Make ``layer``'s weights current in its staging slot on the compute stream (for inspection and tests)."""
        self._wait_gather(layer)
