"""Peer-memory communication for the sharded optimizer step.

The flat gradient and parameter buffers of the engine live in symmetric memory (``torch.distributed.
_symmetric_memory`` does the allocation and the handle exchange; every rank ends up with a device pointer to
every peer's buffer).  The collectives themselves are this repository's kernels (``csrc/comm/rs_optim.cu``):

* ``reduce_scatter_grads``: barrier, then each rank pulls and sums its shard from all peers' gradient buffers.
* ``adamw_and_publish``: AdamW on the shard, with the bf16 result stored into every peer's parameter buffer,
  then a barrier so that no rank starts its next forward (or clears its gradients) before all peers are done
  reading and writing.

Barriers are sequence-numbered flags in a small symmetric buffer with bounded waits: a rank that never shows up
produces a recorded timeout status on the others instead of a hang.
"""

from __future__ import annotations

import os

import torch
import torch.distributed as dist

from mintext_b200.ops._ext import ext, status_word


def multicast_available(handle) -> bool:
    """Whether the symmetric-memory rendezvous bound the buffer to an NVLink multicast object (NVLS): the handle then
    carries a multicast address that `multimem` instructions could use.  This repository's kernels do not (they use
    plain peer loads and stores); the probe only reports what the platform offers, once, at start-up."""
    try:
        return bool(int(getattr(handle, "multicast_ptr", 0) or 0))
    except Exception:
        return False


class SymmetricOptimizerComm:
    def __init__(self, engine):
        import torch.distributed._symmetric_memory as symm

        self.engine = engine
        group = engine.group or dist.group.WORLD
        self.rank, self.world = engine.rank, engine.world
        if self.world > 8:
            raise RuntimeError("the peer-memory optimizer path covers a single NVSwitch domain of at most 8 GPUs")
        self.flags = symm.empty(64, dtype=torch.int32, device=engine.device)
        self.flags.zero_()
        self._h_flags = symm.rendezvous(self.flags, group)
        self._h_grad = symm.rendezvous(engine.grad_flat, group)
        self._h_param = symm.rendezvous(engine.param_flat, group)
        self.flag_ptrs = [int(p) for p in self._h_flags.buffer_ptrs]
        self.grad_ptrs = [int(p) for p in self._h_grad.buffer_ptrs]
        self.param_ptrs = [int(p) for p in self._h_param.buffer_ptrs]
        self.seq = 0
        # per-bucket readiness flags for the overlapped gradient reduction, and the stream it runs on
        self.bucket_slots = int(ext().bucket_flag_slots())
        if len(engine.buckets) > self.bucket_slots:
            raise RuntimeError(f"{len(engine.buckets)} gradient buckets exceed the {self.bucket_slots} flag slots")
        self.bucket_flags = symm.empty(self.world * self.bucket_slots, dtype=torch.int32, device=engine.device)
        self.bucket_flags.zero_()
        self._h_bflags = symm.rendezvous(self.bucket_flags, group)
        self.bflag_ptrs = [int(p) for p in self._h_bflags.buffer_ptrs]
        self.side = torch.cuda.Stream(device=engine.device)
        self.round = 0            # one per optimizer step; flags carry 2 * round (+ 1 for second pulls)
        self._round_open = False
        self.side_blocks = int(os.environ.get("MT_GRAD_PULL_BLOCKS", "32"))
        self.split_handshake = os.environ.get("MT_GRAD_PULL_SPLIT_HANDSHAKE", "1") != "0"
        self.multicast = multicast_available(self._h_grad)
        if self.rank == 0:
            import logging

            logging.getLogger(__name__).info("peer-memory optimizer path: %d ranks, NVLink multicast %s (not used: "
                                             "peer loads / stores only)", self.world,
                                             "available" if self.multicast else "not available")
        torch.cuda.synchronize(engine.device)
        dist.barrier(group=group)  # flags are zeroed everywhere before the first in-kernel barrier

    def barrier(self) -> None:
        self.seq += 1
        ext().symm_barrier(self.flag_ptrs, self.rank, self.seq, status_word(self.engine.device))

    def reduce_scatter_grads(self, out: torch.Tensor) -> None:
        """``out`` <- sum over ranks of their gradient buffers on this rank's shard range; also adds the
        shard's sum of squares into the engine's ``_sumsq``."""
        e = self.engine
        self.barrier()  # every rank's backward has finished writing its gradient buffer
        e._sumsq_shard.zero_()
        ext().grad_pull_reduce(self.grad_ptrs, self.rank, self.rank * e.shard_size, out, e._sumsq_shard)

    # -- bucketed reduction, overlapped with the backward pass ---------------------------------------------------
    def _pull(self, bucket: int, accumulate: bool, blocks: int, split_handshake: bool = False) -> None:
        """``split_handshake``: wait for the peers in a one-warp kernel of its own in front of the reduction, so that
        no multi-block grid sits on SMs while it waits (under the backward pass a waiting block can keep an
        attention-backward block, which needs the whole register file, off its SM)."""
        e = self.engine
        _, a, b, loc = e.segments[bucket]
        seq = 2 * self.round + (1 if accumulate else 0)
        if split_handshake:
            ext().bucket_ready(self.bflag_ptrs, self.rank, bucket, seq, status_word(e.device))
        ext().grad_pull_bucket(self.grad_ptrs, self.bflag_ptrs, self.rank, bucket, seq, a, e.grad_shard[loc:loc + (b - a)],
                               accumulate, True, not split_handshake, blocks, status_word(e.device))

    def _open_round(self) -> None:
        if not self._round_open:
            self.round += 1
            self._round_open = True

    def pull_bucket_async(self, bucket: int) -> None:
        """Called from inside the backward pass once every gradient kernel of ``bucket`` has been launched: the
        bucket's reduction is queued on the side stream behind those kernels, on a few SMs."""
        self._open_round()
        self.side.wait_stream(torch.cuda.current_stream(self.engine.device))
        _, a, b, _ = self.engine.segments[bucket]
        # a few SMs' worth of blocks for a layer of a small model, more for slices of hundreds of megabytes, so that
        # the pull finishes under the rest of the backward pass without crowding it
        blocks = max(self.side_blocks, min(296, (b - a) * 4 // (2 << 20)))
        with torch.cuda.stream(self.side):
            self._pull(bucket, False, blocks, split_handshake=self.split_handshake)

    def wait_side_stream(self) -> None:
        torch.cuda.current_stream(self.engine.device).wait_stream(self.side)

    def finish_bucket_pulls(self, pulled: set, late: set) -> None:
        """After the backward pass: reduce the buckets that were not started early, and run a second, accumulating
        pull for buckets that received gradients after theirs had been issued (the same set on every rank)."""
        self._open_round()
        self.wait_side_stream()
        for b in range(len(self.engine.buckets)):
            if b not in pulled:
                self._pull(b, False, 0)
        for b in sorted(late):
            self._pull(b, True, 0)
        self._round_open = False

    def adamw_and_publish(self, grad_shard: torch.Tensor, lr, bc1, bc2, grad_scale, clip: torch.Tensor) -> None:
        e, cfg = self.engine, self.engine.config
        for _, a, b, loc in e.segments:
            sl = slice(loc, loc + (b - a))
            ext().adamw_publish(e.master[sl], e.exp_avg[sl], e.exp_avg_sq[sl], grad_shard[sl], self.param_ptrs, a,
                                lr, cfg.adam_b1, cfg.adam_b2, cfg.adam_eps, cfg.weight_decay, bc1, bc2, grad_scale, clip)
        self.barrier()  # all shards published everywhere, all peers done reading this rank's gradients


class MuonPublishComm:
    """Publication of Muon's updated bf16 shards without a library collective: every rank owns one contiguous
    ``1/N`` bin of the flat parameter buffer (symmetric memory); after its update it waits at a flag barrier, pulls the
    other ranks' bins from their buffers into its own (``peer_gather``: plain peer loads) and waits again, so that no
    rank overwrites its bin in the next step while a peer still reads it."""

    def __init__(self, engine):
        import torch.distributed._symmetric_memory as symm

        self.engine = engine
        group = engine.group or dist.group.WORLD
        self.rank, self.world = engine.rank, engine.world
        if self.world > 8:
            raise RuntimeError("the peer-memory path covers a single NVSwitch domain of at most 8 GPUs")
        self.flags = symm.empty(64, dtype=torch.int32, device=engine.device)
        self.flags.zero_()
        self._h_flags = symm.rendezvous(self.flags, group)
        self._h_param = symm.rendezvous(engine.param_flat, group)
        self.flag_ptrs = [int(p) for p in self._h_flags.buffer_ptrs]
        self.param_ptrs = [int(p) for p in self._h_param.buffer_ptrs]
        self.seq = 0
        torch.cuda.synchronize(engine.device)
        dist.barrier(group=group)

    def _barrier(self) -> None:
        self.seq += 1
        ext().symm_barrier(self.flag_ptrs, self.rank, self.seq, status_word(self.engine.device))

    def publish(self) -> None:
        e = self.engine
        self._barrier()  # every rank's bin holds its updated weights
        ext().peer_gather(self.param_ptrs, 0, e.shard_size, e.shard_size, e.param_flat, 0)
        self._barrier()  # every rank has read every bin
