"""Expert parallelism on CPU ranks (gloo): the collective exchange reproduces the single-process MoE block,
forward and backward, when every rank holds a slice of the experts and its own tokens."""

import torch
import torch.distributed as dist

from mintext_b200 import MinTextConfig
from tests.test_sharding import run_ranks


def _cfg():
    return MinTextConfig(dtype="float32", hidden_size=32, num_experts=8, num_experts_per_tok=2, moe_intermediate_size=16,
                         n_group=4, topk_group=2, n_shared_experts=1)


def _tokens(rank):
    return torch.randn(12, 32, generator=torch.Generator().manual_seed(100 + rank))


def _ep_worker(rank, world):
    from mintext_b200.modules import MoEBlock
    from mintext_b200.parallel.ep import ExpertParallel, set_current_ep

    set_current_ep(ExpertParallel(dist.group.WORLD, torch.device("cpu"), fused=False))
    try:
        blk = MoEBlock(_cfg(), rngs=torch.Generator().manual_seed(0))
        assert blk.experts.gate_up_proj.shape[0] == 8 // world
        x = _tokens(rank).view(1, 12, 32).requires_grad_(True)
        out, _ = blk(x)
        out.pow(2).sum().backward()
        return (out.detach(), x.grad.clone(), blk.experts.gate_up_proj.grad.clone(), blk.router.gate.kernel.grad.clone())
    finally:
        set_current_ep(None)


def test_collective_expert_parallel_matches_single_process():
    world = 2
    res = run_ranks(_ep_worker, world, 29623)
    from mintext_b200.modules import MoEBlock

    blk = MoEBlock(_cfg(), rngs=torch.Generator().manual_seed(0))
    xs = [_tokens(r).view(1, 12, 32).requires_grad_(True) for r in range(world)]
    outs = [blk(x)[0] for x in xs]
    sum(o.pow(2).sum() for o in outs).backward()
    per = 8 // world
    router_grad = torch.zeros_like(blk.router.gate.kernel)
    for r in range(world):
        out, dx, dgu, dgate = res[r]
        assert torch.allclose(out, outs[r].detach(), atol=1e-5)
        assert torch.allclose(dx, xs[r].grad, atol=1e-5)
        assert torch.allclose(dgu, blk.experts.gate_up_proj.grad[r * per:(r + 1) * per], atol=1e-5)
        router_grad += dgate
    # the router is replicated: its gradient is the sum of the per-rank contributions
    assert torch.allclose(router_grad, blk.router.gate.kernel.grad, atol=1e-5)
