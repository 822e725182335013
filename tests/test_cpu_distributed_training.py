"""Several CPU processes (gloo) train through ``setup_training`` + ``trainer.train_step`` and end with the weights a
single process gets from the same global batches: data parallelism, tensor parallelism (with vocabulary-parallel ends),
expert parallelism and their combination, over several optimizer steps with global-norm clipping."""

import pytest
import torch

from mintext_b200 import MinTextConfig
from tests.test_sharding import run_ranks

STEPS = 3
BASE = dict(dtype="float32", vocab_size=64, num_hidden_layers=2, hidden_size=32, num_attention_heads=4,
            num_key_value_heads=2, intermediate_size=64, seq_length=16, use_qk_norm=True, model_type="qwen3",
            kernel_backend="oracle", enable_tensorboard=False, enable_checkpointing=False, learning_rate=1e-2,
            gradient_clip_threshold=0.5, per_device_batch_size=2, steps=STEPS, warmup_steps_fraction=0.0)
MOE = dict(model_type="deepseek_v3", use_qk_norm=False, num_experts=4, num_experts_per_tok=2, moe_intermediate_size=16,
           n_group=2, topk_group=1, first_k_dense_replace=1, n_shared_experts=1, moe_capacity_factor=8.0)
CASES = {
    # name: (ranks, parallelism, extra model settings)
    "data_parallel": (2, dict(ici_fsdp_parallelism=2), {}),
    "data_parallel_with_accumulation": (2, dict(ici_data_parallelism=2), dict(gradient_accumulation_steps=2)),
    "tensor_and_vocab_parallel": (4, dict(ici_fsdp_parallelism=2, ici_tensor_parallelism=2),
                                  dict(tp_vocab_parallel=True, z_loss_weight=1e-3)),
    "expert_parallel": (2, dict(ici_fsdp_parallelism=2, ici_expert_parallelism=2), MOE),
    "tensor_and_expert_parallel": (4, dict(ici_fsdp_parallelism=2, ici_tensor_parallelism=2, ici_expert_parallelism=2),
                                   MOE),
    # Muon on sliced matrices: the Newton-Schulz Gram matrices are summed over the tensor-parallel group
    "muon_on_tensor_parallel_slices": (4, dict(ici_fsdp_parallelism=2, ici_tensor_parallelism=2),
                                       dict(optimizer="muon", tp_vocab_parallel=True, learning_rate=2e-3)),
    # two slices (nodes) of four ranks: data parallel across them, fsdp x tensor inside each
    "two_slices": (8, dict(num_slices=2, dcn_data_parallelism=2, ici_fsdp_parallelism=2, ici_tensor_parallelism=2), {}),
}


def _config(case: str, parallel: bool) -> MinTextConfig:
    ranks, par, extra = CASES[case]
    cfg = dict(BASE, **extra)
    if parallel:
        cfg.update(par)
    else:  # one process sees the whole global batch
        dp = ranks // par.get("ici_tensor_parallelism", 1)
        cfg["per_device_batch_size"] = BASE["per_device_batch_size"] * dp
    return MinTextConfig(**cfg)


def _global_batches(case: str):
    ranks, par, _ = CASES[case]
    accum = CASES[case][2].get("gradient_accumulation_steps", 1)
    rows = BASE["per_device_batch_size"] * accum * (ranks // par.get("ici_tensor_parallelism", 1))
    g = torch.Generator().manual_seed(11)
    out = []
    for _ in range(STEPS):
        t = torch.randint(0, 64, (rows, 16), generator=g)
        out.append({"input_tokens": t, "target_tokens": t.roll(-1, 1)})
    return out


def _train_worker(rank, world, case):
    from mintext_b200 import trainer
    from mintext_b200.parallel.ep import set_current_ep
    from mintext_b200.parallel.tp import set_current_tp
    from mintext_b200.train import setup_training

    cfg = _config(case, parallel=True)
    try:
        mesh, model, state, device, use_gpu = setup_training(cfg)
        assert not use_gpu and state.groups is not None
        tp = mesh.shape["tensor"]
        b = cfg.per_device_batch_size * cfg.gradient_accumulation_steps
        dp = rank // tp
        log = []
        for batch in _global_batches(case):
            mine = {k: v[dp * b:(dp + 1) * b] for k, v in batch.items()}
            state, m = trainer.train_step(state, mine, model, cfg)
            if m.get("moe_expert_counts") is not None:
                state = trainer.update_expert_biases(state, m["moe_expert_counts"], cfg)
            log.append((float(m["loss"]), float(m["grad_norm"]), float(m["param_norm"])))
        params = {n: (p.detach().clone(), tuple(getattr(p, "shard_spec", ()))) for n, p in model.named_parameters()}
        return log, params
    finally:
        set_current_tp(None)
        set_current_ep(None)


def _worker(case):
    # run_ranks pickles the function: module-level closures per case
    return globals()[f"_worker_{case}"]


def _worker_data_parallel(rank, world):
    return _train_worker(rank, world, "data_parallel")


def _worker_data_parallel_with_accumulation(rank, world):
    return _train_worker(rank, world, "data_parallel_with_accumulation")


def _worker_tensor_and_vocab_parallel(rank, world):
    return _train_worker(rank, world, "tensor_and_vocab_parallel")


def _worker_expert_parallel(rank, world):
    return _train_worker(rank, world, "expert_parallel")


def _worker_tensor_and_expert_parallel(rank, world):
    return _train_worker(rank, world, "tensor_and_expert_parallel")


def _worker_muon_on_tensor_parallel_slices(rank, world):
    return _train_worker(rank, world, "muon_on_tensor_parallel_slices")


def _worker_two_slices(rank, world):
    return _train_worker(rank, world, "two_slices")


def _single_process(case):
    from mintext_b200 import trainer
    from mintext_b200.train import setup_training

    cfg = _config(case, parallel=False)
    mesh, model, state, device, use_gpu = setup_training(cfg)
    assert state.groups is None
    log = []
    for batch in _global_batches(case):
        state, m = trainer.train_step(state, batch, model, cfg)
        if m.get("moe_expert_counts") is not None:
            state = trainer.update_expert_biases(state, m["moe_expert_counts"], cfg)
        log.append((float(m["loss"]), float(m["grad_norm"]), float(m["param_norm"])))
    return log, {n: p.detach().clone() for n, p in model.named_parameters()}


@pytest.mark.parametrize("case,port", [("data_parallel", 29661), ("data_parallel_with_accumulation", 29673),
                                       ("tensor_and_vocab_parallel", 29663),
                                       ("expert_parallel", 29665), ("tensor_and_expert_parallel", 29667),
                                       ("two_slices", 29671), ("muon_on_tensor_parallel_slices", 29675)])
def test_cpu_processes_train_to_the_single_process_weights(case, port):
    ranks = CASES[case][0]
    res = run_ranks(_worker(case), ranks, port)
    ref_log, ref = _single_process(case)
    for r in range(ranks):
        for got, want in zip(res[r][0], ref_log):   # loss, gradient norm and parameter norm of every step
            assert got == pytest.approx(want, rel=2e-4, abs=2e-5), (case, r, res[r][0], ref_log)
    for name, full in ref.items():
        pieces = {}
        for r in range(ranks):
            t, spec = res[r][1][name]
            if not spec:
                assert torch.allclose(t, full, atol=2e-5), (case, name, r, float((t - full).abs().max()))
                continue
            dim, idx, cnt = spec
            if idx in pieces:  # replicas of one slice hold the same values
                assert torch.allclose(t, pieces[idx][1], atol=1e-6), (case, name, r)
            pieces[idx] = (dim, t)
        if pieces:
            dim = next(iter(pieces.values()))[0]
            got = torch.cat([pieces[i][1] for i in sorted(pieces)], dim=dim)
            assert got.shape == full.shape and torch.allclose(got, full, atol=2e-5), \
                (case, name, float((got - full).abs().max()))


# ------------------------------------------------------------------ checkpoints of sliced parameters
def _ckpt_worker(rank, world):
    """Two steps on 4 ranks (fsdp 2 x tensor 2, vocabulary-parallel), save, one more step; then restore the saved
    step into the same layout and repeat the third step: same weights."""
    import os

    from mintext_b200 import trainer
    from mintext_b200.checkpoint import CheckpointManager
    from mintext_b200.parallel.tp import set_current_tp
    from mintext_b200.train import setup_training

    case = "tensor_and_vocab_parallel"
    cfg = _config(case, parallel=True)
    try:
        mesh, model, state, _, _ = setup_training(cfg)
        b, dp = cfg.per_device_batch_size, rank // mesh.shape["tensor"]
        batches = [{k: v[dp * b:(dp + 1) * b] for k, v in gb.items()} for gb in _global_batches(case)]
        for mine in batches[:2]:
            state, _ = trainer.train_step(state, mine, model, cfg)
        mgr = CheckpointManager(os.environ["MT_TEST_CKPT_DIR"], save_interval_steps=1, max_to_keep=2, enable_async=False)
        assert mgr.save(2, state, force=True)
        mgr.wait_until_finished()
        state, _ = trainer.train_step(state, batches[2], model, cfg)
        after3 = {n: p.detach().clone() for n, p in model.named_parameters()}
        mgr.restore(2, state)
        assert state.step == 2
        state, _ = trainer.train_step(state, batches[2], model, cfg)
        for n, p in model.named_parameters():
            assert torch.allclose(p, after3[n], atol=1e-7), n
        return True
    finally:
        set_current_tp(None)


def test_sliced_parameters_checkpoint_on_four_cpu_ranks_and_restore_in_one_process(tmp_path, monkeypatch):
    from mintext_b200 import trainer
    from mintext_b200.checkpoint import CheckpointManager
    from mintext_b200.train import setup_training

    monkeypatch.setenv("MT_TEST_CKPT_DIR", str(tmp_path))
    assert all(run_ranks(_ckpt_worker, 4, 29669).values())
    files = sorted(p.name for p in (tmp_path / "2" / "default").iterdir())
    assert "params__token_embedder.shard0of2.bin" in files and "params__token_embedder.shard1of2.bin" in files
    assert "params__final_norm.scale.bin" in files
    # one process restores the whole tensors from the shards and continues as the four ranks did
    case = "tensor_and_vocab_parallel"
    cfg = _config(case, parallel=False)
    _, model, state, _, _ = setup_training(cfg)
    CheckpointManager(str(tmp_path), save_interval_steps=1, max_to_keep=2, enable_async=False).restore(2, state)
    assert state.step == 2
    ref_cfg = cfg
    _, ref_model, ref_state, _, _ = setup_training(ref_cfg)
    batches = _global_batches(case)
    for gb in batches[:2]:
        ref_state, _ = trainer.train_step(ref_state, gb, ref_model, ref_cfg)
    for (n, p), (_, q) in zip(model.named_parameters(), ref_model.named_parameters()):
        assert torch.allclose(p, q, atol=2e-5), (n, float((p - q).abs().max()))
    state, m = trainer.train_step(state, batches[2], model, cfg)
    ref_state, mr = trainer.train_step(ref_state, batches[2], ref_model, ref_cfg)
    assert float(m["loss"]) == pytest.approx(float(mr["loss"]), rel=1e-4)
