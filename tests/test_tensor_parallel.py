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


MIXED = {
    "deepseek": dict(model_type="deepseek_v3", attention_type="mla", q_lora_rank=16, kv_lora_rank=16, qk_nope_head_dim=8,
                     qk_rope_head_dim=8, v_head_dim=8, num_experts=4, num_experts_per_tok=2, moe_intermediate_size=16,
                     n_group=2, topk_group=1, first_k_dense_replace=1, n_shared_experts=1),
    "qwen3_next": dict(model_type="qwen3_next", use_qk_norm=True, full_attention_interval=2, partial_rotary_factor=0.5,
                       linear_key_head_dim=8, linear_value_head_dim=8, linear_num_key_heads=2, linear_num_value_heads=4,
                       num_experts=4, num_experts_per_tok=2, moe_intermediate_size=16, n_group=1, topk_group=1,
                       first_k_dense_replace=0, router_type="softmax_topk", shared_expert_gate=True, n_shared_experts=1,
                       router_aux_loss_coef=0.05),
}


def _mixed_cfg(kind):
    return MinTextConfig(dtype="float32", vocab_size=64, num_hidden_layers=2, hidden_size=32, num_attention_heads=4,
                         num_key_value_heads=2, intermediate_size=64, seq_length=16, **MIXED[kind])


def _mixed_worker(rank, world, kind):
    from mintext_b200 import trainer
    from mintext_b200.models import Transformer
    from mintext_b200.parallel.tp import TensorParallel, set_current_tp

    set_current_tp(TensorParallel(dist.group.WORLD, torch.device("cpu"), fused=False))
    try:
        cfg = _mixed_cfg(kind)
        m = Transformer(cfg, rngs=0)
        loss, _ = trainer.compute_loss(None, m, cfg, _batch())
        named = [(n, p) for n, p in m.named_parameters() if p.requires_grad]
        grads = torch.autograd.grad(loss, [p for _, p in named], allow_unused=True)
        rep = {n for n, p in named if getattr(p, "tp_replicated_compute", False)}
        return float(loss), {n: (g.clone() if g is not None else None) for (n, _), g in zip(named, grads)}, rep
    finally:
        set_current_tp(None)


def _deepseek_worker(rank, world):
    return _mixed_worker(rank, world, "deepseek")


def _qwen3_next_worker(rank, world):
    return _mixed_worker(rank, world, "qwen3_next")


def _check_mixed(kind, worker, port):
    """Attention variants shard their heads, routers and routed experts work on each rank's token shard (their
    gradients are per-shard contributions like a norm scale's), shared experts shard their hidden columns.  Together
    they give the single-process gradient of mean loss (+ auxiliary loss).  A sub-layer computed in full on every rank
    (none at present) would show identical gradients that count once after the engine's 1/tp scaling."""
    from mintext_b200 import trainer
    from mintext_b200.models import Transformer

    world = 2
    res = run_ranks(worker, world, port)
    cfg = _mixed_cfg(kind)
    m = Transformer(cfg, rngs=0)
    loss, _ = trainer.compute_loss(None, m, cfg, _batch())
    named = [(n, p) for n, p in m.named_parameters() if p.requires_grad]
    ref = dict(zip([n for n, _ in named], torch.autograd.grad(loss, [p for _, p in named], allow_unused=True)))
    replicated = res[0][2]
    assert not replicated, f"no sub-layer should need the replicated fallback: {sorted(replicated)}"
    for name, g in ref.items():
        parts = [res[r][1][name] for r in range(world)]
        if g is None:
            assert all(p is None for p in parts), name
            continue
        if name in replicated:
            assert torch.allclose(parts[0], parts[1], atol=1e-5), name      # identical on every rank
            got = sum(parts) / world / world                                 # engine: 1/tp, then the mean over ranks
        elif parts[0].shape == g.shape:
            got = sum(parts) / world
        else:
            dim = next(i for i, (a, b) in enumerate(zip(parts[0].shape, g.shape)) if a != b)
            got = torch.cat(parts, dim=dim) / world
        assert torch.allclose(got, g, atol=5e-5), (name, (got - g).abs().max())


def test_tensor_parallel_with_head_sharded_mla_and_token_sharded_experts():
    _check_mixed("deepseek", _deepseek_worker, 29633)


def test_tensor_parallel_with_head_sharded_gdn_token_sharded_experts_and_aux_loss():
    _check_mixed("qwen3_next", _qwen3_next_worker, 29635)


def _mla_cfg():
    return MinTextConfig(dtype="float32", vocab_size=64, num_hidden_layers=2, hidden_size=32, num_attention_heads=4,
                         intermediate_size=64, seq_length=16, model_type="deepseek_v3", attention_type="mla",
                         q_lora_rank=16, kv_lora_rank=16, qk_nope_head_dim=8, qk_rope_head_dim=4, v_head_dim=8)


def _mla_tp_worker(rank, world):
    from mintext_b200 import trainer
    from mintext_b200.models import Transformer
    from mintext_b200.parallel.tp import TensorParallel, set_current_tp

    set_current_tp(TensorParallel(dist.group.WORLD, torch.device("cpu"), fused=False))
    try:
        cfg = _mla_cfg()
        m = Transformer(cfg, rngs=0)
        att = m.layers[0].attention
        assert att.q_b_proj.kernel.shape == (16, 2, 12) and att.kv_b_proj.kernel.shape == (16, 2, 16)
        assert att.out.kernel.shape == (2, 8, 32) and att.q_a_proj.kernel.shape == (32, 16)
        assert not getattr(att.q_a_proj.kernel, "tp_replicated_compute", False)
        loss, _ = trainer.compute_loss(None, m, cfg, _batch())
        names = [n for n, _ in m.named_parameters()]
        grads = torch.autograd.grad(loss, list(m.parameters()))
        return float(loss), {n: g.clone() for n, g in zip(names, grads)}
    finally:
        set_current_tp(None)


def test_head_sharded_mla_matches_single_process():
    """Multi-head-latent attention with its heads split over two ranks: the loss and every gradient equal the
    single-process model's (whole low-rank projections collect partial sums, one per rank's heads)."""
    from mintext_b200 import trainer
    from mintext_b200.models import Transformer

    world = 2
    res = run_ranks(_mla_tp_worker, world, 29633)
    cfg = _mla_cfg()
    m = Transformer(cfg, rngs=0)
    loss, _ = trainer.compute_loss(None, m, cfg, _batch())
    ref = dict(zip([n for n, _ in m.named_parameters()], torch.autograd.grad(loss, list(m.parameters()))))
    assert abs(sum(res[r][0] for r in range(world)) / world - float(loss)) < 1e-5
    for name, g in ref.items():
        parts = [res[r][1][name] for r in range(world)]
        if parts[0].shape == g.shape:
            got = sum(parts) / world
        else:
            dim = next(i for i, (a, b) in enumerate(zip(parts[0].shape, g.shape)) if a != b)
            got = torch.cat(parts, dim=dim) / world
        assert torch.allclose(got, g, atol=2e-5), name


def _gdn_cfg():
    return MinTextConfig(dtype="float32", vocab_size=64, num_hidden_layers=2, hidden_size=32, num_attention_heads=4,
                         num_key_value_heads=2, intermediate_size=64, seq_length=16, model_type="qwen3_next",
                         use_qk_norm=True, full_attention_interval=2, partial_rotary_factor=0.5, linear_key_head_dim=8,
                         linear_value_head_dim=8, linear_num_key_heads=2, linear_num_value_heads=4)


def _gdn_tp_worker(rank, world):
    from mintext_b200 import trainer
    from mintext_b200.models import Transformer
    from mintext_b200.parallel.tp import TensorParallel, set_current_tp

    set_current_tp(TensorParallel(dist.group.WORLD, torch.device("cpu"), fused=False))
    try:
        cfg = _gdn_cfg()
        m = Transformer(cfg, rngs=0)
        att = m.layers[0].attention
        # one of two key heads (with its two value heads) per rank: q 8 + k 8 + v 16 + z 16 columns, 2 x (b, a), 16 rows
        assert att.in_proj_qkvz.kernel.shape == (32, 48) and att.in_proj_ba.kernel.shape == (32, 4)
        assert att.out_proj.kernel.shape == (16, 32)
        assert att.conv_weight.shape[0] == 2 * 16 + 32 and att.A_log.shape == (4,)   # whole on every rank
        assert not any(getattr(p, "tp_replicated_compute", False) for p in m.parameters())
        loss, _ = trainer.compute_loss(None, m, cfg, _batch())
        names = [n for n, _ in m.named_parameters()]
        grads = torch.autograd.grad(loss, list(m.parameters()))
        return float(loss), {n: g.clone() for n, g in zip(names, grads)}
    finally:
        set_current_tp(None)


def test_head_sharded_gated_delta_rule_matches_single_process():
    """Gated Delta Rule layers with their key heads (and value-head groups) split over two ranks: the loss and every
    gradient equal the single-process model's; conv weights, A_log, dt_bias and the output norm stay whole and collect
    one partial sum per rank's heads."""
    from mintext_b200 import trainer
    from mintext_b200.models import Transformer

    world = 2
    res = run_ranks(_gdn_tp_worker, world, 29637)
    cfg = _gdn_cfg()
    m = Transformer(cfg, rngs=0)
    loss, _ = trainer.compute_loss(None, m, cfg, _batch())
    ref = dict(zip([n for n, _ in m.named_parameters()], torch.autograd.grad(loss, list(m.parameters()))))
    assert abs(sum(res[r][0] for r in range(world)) / world - float(loss)) < 1e-5
    for name, g in ref.items():
        parts = [res[r][1][name] for r in range(world)]
        if parts[0].shape == g.shape:
            got = sum(parts) / world
        else:
            dim = next(i for i, (a, b) in enumerate(zip(parts[0].shape, g.shape)) if a != b)
            got = torch.cat(parts, dim=dim) / world
        assert torch.allclose(got, g, atol=2e-5), (name, float((got - g).abs().max()))


def _tp_ep_cfg():
    return MinTextConfig(dtype="float32", vocab_size=64, num_hidden_layers=2, hidden_size=32, num_attention_heads=4,
                         num_key_value_heads=2, intermediate_size=64, seq_length=16, model_type="deepseek_v3",
                         attention_type="mla", q_lora_rank=16, kv_lora_rank=16, qk_nope_head_dim=8, qk_rope_head_dim=8,
                         v_head_dim=8, num_experts=4, num_experts_per_tok=2, moe_intermediate_size=16, n_group=2,
                         topk_group=1, first_k_dense_replace=1, n_shared_experts=1, ici_fsdp_parallelism=2,
                         ici_tensor_parallelism=2, ici_expert_parallelism=2)


def _global_batch():
    t = torch.randint(0, 64, (4, 16), generator=torch.Generator().manual_seed(5))
    return {"input_tokens": t, "target_tokens": t.roll(-1, 1)}


def _tp_ep_worker(rank, world):
    """4 ranks = 2 data-parallel groups x 2 tensor-parallel ranks; experts split over the 2 ranks of each tensor
    column (expert parallelism inside the data-parallel ranks)."""
    from mintext_b200 import trainer
    from mintext_b200.models import Transformer
    from mintext_b200.parallel.ep import ExpertParallel, set_current_ep
    from mintext_b200.parallel.mesh import create_mesh
    from mintext_b200.parallel.tp import TensorParallel, set_current_tp

    cfg = _tp_ep_cfg()
    mesh = create_mesh(cfg)
    set_current_ep(ExpertParallel(mesh.group(("expert",)), torch.device("cpu"), fused=False))
    set_current_tp(TensorParallel(mesh.group(("tensor",)), torch.device("cpu"), fused=False))
    try:
        m = Transformer(cfg, rngs=0)
        assert m.layers[1].mlp.experts.gate_up_proj.shape[0] == 2          # half of the experts
        assert m.layers[1].mlp.shared_expert.gate.kernel.shape == (32, 8)  # half of the shared expert's columns
        dp = rank // 2
        b = {k: v[2 * dp:2 * dp + 2] for k, v in _global_batch().items()}
        loss, _ = trainer.compute_loss(None, m, cfg, b)
        named = [(n, p) for n, p in m.named_parameters() if p.requires_grad]
        grads = torch.autograd.grad(loss, [p for _, p in named], allow_unused=True)
        return float(loss), {n: (g.clone() if g is not None else None) for (n, _), g in zip(named, grads)}
    finally:
        set_current_tp(None)
        set_current_ep(None)


def test_tensor_and_expert_parallelism_together_match_single_process():
    """Token-sharded tensor parallelism with the routed experts split over the data-parallel ranks of each tensor
    column: the mean of the ranks' losses and the assembled gradients equal the single-process model on the global
    batch (expert slices are replicated across the tensor axis, tensor slices across the data axis)."""
    from mintext_b200 import trainer
    from mintext_b200.models import Transformer

    res = run_ranks(_tp_ep_worker, 4, 29641)
    cfg = _tp_ep_cfg().model_copy(update={"ici_fsdp_parallelism": 1, "ici_tensor_parallelism": 1,
                                          "ici_expert_parallelism": 1})
    m = Transformer(cfg, rngs=0)
    loss, _ = trainer.compute_loss(None, m, cfg, _global_batch())
    named = [(n, p) for n, p in m.named_parameters() if p.requires_grad]
    ref = dict(zip([n for n, _ in named], torch.autograd.grad(loss, [p for _, p in named], allow_unused=True)))
    assert abs(sum(res[r][0] for r in range(4)) / 4 - float(loss)) < 1e-5
    rank_of = lambda dp, j: 2 * dp + j
    for name, g in ref.items():
        parts = [res[r][1][name] for r in range(4)]
        if g is None:
            assert all(p is None for p in parts), name
            continue
        if parts[0].shape == g.shape:                       # whole on every rank: per-rank contributions
            got = sum(parts) / 4
        elif ".experts." in name:                           # expert block p lives on data rank p of both tensor columns
            got = torch.cat([sum(parts[rank_of(p, j)] for j in range(2)) / 4 for p in range(2)], dim=0)
        else:                                               # tensor slice j lives on tensor rank j of both data ranks
            dim = next(i for i, (a, b) in enumerate(zip(parts[0].shape, g.shape)) if a != b)
            got = torch.cat([sum(parts[rank_of(dp, j)] for dp in range(2)) / 4 for j in range(2)], dim=dim)
        assert torch.allclose(got, g, atol=5e-5), (name, float((got - g).abs().max()))


def _setup_training_worker(rank, world):
    """``setup_training`` on 4 CPU ranks with tensor x expert parallelism: contexts, replica groups, model; then one
    loss evaluation through the trainer."""
    from mintext_b200 import trainer
    from mintext_b200.parallel.ep import current_ep, set_current_ep
    from mintext_b200.parallel.tp import current_tp, set_current_tp
    from mintext_b200.train import setup_training

    cfg = _tp_ep_cfg().model_copy(update={"kernel_backend": "oracle", "enable_tensorboard": False,
                                          "enable_checkpointing": False})
    try:
        mesh, model, state, device, use_gpu = setup_training(cfg)
        assert not use_gpu and device.type == "cpu"
        assert current_tp().size == 2 and current_ep().size == 2
        assert dict(mesh.shape) == {"data": 1, "fsdp": 2, "tensor": 2, "expert": 2}
        dp = rank // 2
        b = {k: v[2 * dp:2 * dp + 2] for k, v in _global_batch().items()}
        loss, _ = trainer.compute_loss(None, model, cfg, b)
        return float(loss)
    finally:
        set_current_tp(None)
        set_current_ep(None)


def test_setup_training_builds_tensor_and_expert_contexts_together():
    from mintext_b200 import trainer
    from mintext_b200.models import Transformer

    res = run_ranks(_setup_training_worker, 4, 29645)
    cfg = _tp_ep_cfg().model_copy(update={"ici_fsdp_parallelism": 1, "ici_tensor_parallelism": 1,
                                          "ici_expert_parallelism": 1})
    loss, _ = trainer.compute_loss(None, Transformer(cfg, rngs=0), cfg, _global_batch())
    assert abs(sum(res.values()) / 4 - float(loss)) < 1e-5


VOCAB_PARALLEL = {
    "plain": dict(),
    "tied_smoothing_zloss": dict(tie_word_embeddings=True, label_smoothing=0.1, z_loss_weight=1e-3, num_vocab_tiles=3),
    "softcap_scaled": dict(final_logit_softcapping=5.0, scale_embeddings=True, z_loss_weight=1e-3,
                           num_key_value_heads=4),
}


def _vp_cfg(kind):
    return _cfg().model_copy(update=dict(tp_vocab_parallel=True, **VOCAB_PARALLEL[kind]))


def _vp_worker(rank, world, kind):
    from mintext_b200 import trainer
    from mintext_b200.models import Transformer
    from mintext_b200.parallel.tp import TensorParallel, set_current_tp

    set_current_tp(TensorParallel(dist.group.WORLD, torch.device("cpu"), fused=False))
    try:
        cfg = _vp_cfg(kind)
        m = Transformer(cfg, rngs=0)
        assert m.vocab_parallel and m.token_embedder.shape == (64 // world, 32)
        assert m.token_embedder.shard_spec == (0, rank, world) and m.token_embedder.tensor_parallel
        if not cfg.tie_word_embeddings:
            assert m.output_proj.kernel.shape == (32, 64 // world) and m.output_proj.kernel.shard_spec == (1, rank, world)
        loss, aux = trainer.compute_loss(None, m, cfg, _batch())
        names = [n for n, _ in m.named_parameters()]
        grads = torch.autograd.grad(loss, list(m.parameters()))
        return float(loss), {n: g.clone() for n, g in zip(names, grads)}, float(aux["z_loss"])
    finally:
        set_current_tp(None)


def _vp_plain(rank, world):
    return _vp_worker(rank, world, "plain")


def _vp_tied(rank, world):
    return _vp_worker(rank, world, "tied_smoothing_zloss")


def _vp_softcap(rank, world):
    return _vp_worker(rank, world, "softcap_scaled")


def _check_vocab_parallel(kind, worker, world, port):
    from mintext_b200 import trainer
    from mintext_b200.models import Transformer

    res = run_ranks(worker, world, port)
    cfg = _vp_cfg(kind).model_copy(update={"tp_vocab_parallel": False})
    m = Transformer(cfg, rngs=0)
    loss, aux = trainer.compute_loss(None, m, cfg, _batch())
    ref = dict(zip([n for n, _ in m.named_parameters()], torch.autograd.grad(loss, list(m.parameters()))))
    assert abs(sum(res[r][0] for r in range(world)) / world - float(loss)) < 1e-5
    assert abs(sum(res[r][2] for r in range(world)) / world - float(aux["z_loss"])) < 1e-6
    for name, g in ref.items():
        parts = [res[r][1][name] for r in range(world)]
        if parts[0].shape == g.shape:
            got = sum(parts) / world
        else:
            dim = next(i for i, (a, b) in enumerate(zip(parts[0].shape, g.shape)) if a != b)
            got = torch.cat(parts, dim=dim) / world
        assert torch.allclose(got, g, atol=2e-5), (name, (got - g).abs().max())
    for name in ("token_embedder",) + (() if cfg.tie_word_embeddings else ("output_proj.kernel",)):
        assert res[0][1][name].shape != ref[name].shape, f"{name} should be sharded over the vocabulary"


def test_vocab_parallel_embedding_and_head_match_single_process():
    _check_vocab_parallel("plain", _vp_plain, 2, 29651)


def test_vocab_parallel_tied_weights_label_smoothing_z_loss_and_token_chunks():
    _check_vocab_parallel("tied_smoothing_zloss", _vp_tied, 2, 29653)


def test_vocab_parallel_soft_capped_logits_on_four_ranks():
    _check_vocab_parallel("softcap_scaled", _vp_softcap, 4, 29655)


def _vp_embedding_worker(rank, world):
    """bf16 table: the reduce-scatter adds one non-zero row and zeros per token, so the result is the plain lookup."""
    from mintext_b200.parallel import vocab_parallel as vp
    from mintext_b200.parallel.tp import TensorParallel

    tp = TensorParallel(dist.group.WORLD, torch.device("cpu"), fused=False)
    g = torch.Generator().manual_seed(5)
    table = torch.randn(64, 16, generator=g).to(torch.bfloat16)
    tokens = torch.randint(0, 64, (1, 8 * world), generator=g)
    per = 64 // world
    local = table[rank * per:(rank + 1) * per].clone().requires_grad_(True)
    mine = tokens[:, rank * 8:(rank + 1) * 8]
    x = vp.embedding(local, mine, tp, torch.bfloat16, scale=2.0)
    assert torch.equal(x, (table[mine] * 2.0).to(torch.bfloat16))
    x.float().sum().backward()
    # every occurrence of a row in the group's tokens adds `scale` to each of its elements
    counts = torch.bincount(tokens.reshape(-1), minlength=64)[rank * per:(rank + 1) * per]
    assert torch.equal(local.grad.float(), (counts[:, None] * 2.0).expand(-1, 16).to(torch.float32))
    return True


def test_vocab_parallel_embedding_is_an_exact_lookup_in_bf16():
    assert all(run_ranks(_vp_embedding_worker, 4, 29657).values())


def _vp_bf16_worker(rank, world):
    """bf16 hidden states and head (the GPU engine's dtypes): loss close to the fp32 oracle, gradient dtypes kept."""
    from mintext_b200.ops import oracle
    from mintext_b200.parallel import vocab_parallel as vp
    from mintext_b200.parallel.tp import TensorParallel

    tp = TensorParallel(dist.group.WORLD, torch.device("cpu"), fused=False)
    g = torch.Generator().manual_seed(9)
    h_all = (torch.randn(8 * world, 32, generator=g) * 0.5).to(torch.bfloat16)
    w_all = (torch.randn(32, 96, generator=g) / 6).to(torch.bfloat16)
    t_all = torch.randint(0, 96, (8 * world,), generator=g)
    per = 96 // world
    h = h_all[rank * 8:(rank + 1) * 8].clone().requires_grad_(True)
    w = w_all[:, rank * per:(rank + 1) * per].clone().requires_grad_(True)
    loss, z = vp.linear_cross_entropy(h, w, t_all[rank * 8:(rank + 1) * 8], tp, False, 0.05, 1e-3, None, chunks=3)
    loss.sum().backward()
    assert h.grad.dtype == torch.bfloat16 and w.grad.dtype == torch.bfloat16 and w.grad.shape == w.shape
    ref, zref = oracle.cross_entropy((h_all.float() @ w_all.float()), t_all, 0.05, 1e-3)
    sl = slice(rank * 8, (rank + 1) * 8)
    return float((loss - ref[sl]).abs().max()), float((z - zref[sl]).abs().max())


def test_vocab_parallel_loss_in_bf16_stays_close_to_the_fp32_oracle():
    res = run_ranks(_vp_bf16_worker, 2, 29659)
    for err, zerr in res.values():
        assert err < 3e-2 and zerr < 1e-3
