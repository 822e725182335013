"""Tensor parallelism on CPU ranks (gloo): token-sharded activations with column / row parallel projections give
the loss and the gradients of the single-process model."""

import torch
import torch.distributed as dist

from mintext_b200 import MinTextConfig
from tests.test_sharding import run_ranks


def _cfg():
    return MinTextConfig(dtype="float32", vocab_size=64, num_hidden_layers=2, hidden_size=32, num_attention_heads=4,
                         num_key_value_heads=2, intermediate_size=64, seq_length=16, use_qk_norm=True,
                         model_type="qwen3")


def _batch():
    t = torch.randint(0, 64, (2, 16), generator=torch.Generator().manual_seed(3))
    return {"input_tokens": t, "target_tokens": t.roll(-1, 1)}


def _tp_worker(rank, world):
    from mintext_b200 import trainer
    from mintext_b200.models import Transformer
    from mintext_b200.parallel.tp import TensorParallel, set_current_tp

    set_current_tp(TensorParallel(dist.group.WORLD, torch.device("cpu"), fused=False))
    try:
        cfg = _cfg()
        m = Transformer(cfg, rngs=0)
        assert m.layers[0].attention.query.kernel.shape == (32, 2, 8)
        assert m.layers[0].mlp.gate.kernel.shape == (32, 32)
        loss, _ = trainer.compute_loss(None, m, cfg, _batch())
        names = [n for n, _ in m.named_parameters()]
        grads = torch.autograd.grad(loss, list(m.parameters()))
        return float(loss), {n: g.clone() for n, g in zip(names, grads)}
    finally:
        set_current_tp(None)


def test_tensor_parallel_matches_single_process():
    from mintext_b200 import trainer
    from mintext_b200.models import Transformer

    world = 2
    res = run_ranks(_tp_worker, world, 29631)
    cfg = _cfg()
    m = Transformer(cfg, rngs=0)
    loss, _ = trainer.compute_loss(None, m, cfg, _batch())
    ref = dict(zip([n for n, _ in m.named_parameters()], torch.autograd.grad(loss, list(m.parameters()))))
    assert abs(sum(res[r][0] for r in range(world)) / world - float(loss)) < 1e-5
    for name, g in ref.items():
        parts = [res[r][1][name] for r in range(world)]
        if parts[0].shape == g.shape:  # replicated parameter: ranks hold per-token-shard contributions
            got = sum(parts) / world
        else:  # sharded parameter: concatenate the slices along the sharded dim
            dim = next(i for i, (a, b) in enumerate(zip(parts[0].shape, g.shape)) if a != b)
            got = torch.cat(parts, dim=dim) / world
        assert torch.allclose(got, g, atol=2e-5), name
