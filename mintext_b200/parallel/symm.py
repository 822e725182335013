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

import torch
import torch.distributed as dist

from mintext_b200.ops._ext import ext, status_word


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

    def adamw_and_publish(self, grad_shard: torch.Tensor, lr, bc1, bc2, grad_scale, clip: torch.Tensor) -> None:
        e, cfg = self.engine, self.engine.config
        ext().adamw_publish(e.master, e.exp_avg, e.exp_avg_sq, grad_shard, self.param_ptrs, self.rank * e.shard_size,
                            lr, cfg.adam_b1, cfg.adam_b2, cfg.adam_eps, cfg.weight_decay, bc1, bc2, grad_scale, clip)
        self.barrier()  # all shards published everywhere, all peers done reading this rank's gradients
