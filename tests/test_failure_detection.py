"""Failure detection without touching a GPU: heartbeats over a store (a rank that stops, a rank that never joins),
gloo ranks where one leaves between steps, the non-finite-loss policies, and damaged checkpoints."""

import time

import pytest
import torch
import torch.distributed as dist

from mintext_b200 import MinTextConfig
from mintext_b200.parallel.health import Heartbeat, NonFiniteLoss, PeerFailure, apply_nan_policy
from tests.test_sharding import run_ranks


def test_heartbeat_detects_a_rank_that_stops():
    store = dist.HashStore()
    a = Heartbeat(store, 0, 2, interval_s=0.05, timeout_s=0.4)
    b = Heartbeat(store, 1, 2, interval_s=0.05, timeout_s=0.4)
    try:
        a.wait_all_alive(2.0)
        a.check()
        time.sleep(0.2)
        a.check()  # both alive
        b.close()  # rank 1 "dies": its counter stops advancing
        a.check()  # records the last value seen
        time.sleep(0.6)
        with pytest.raises(PeerFailure, match=r"rank\(s\) \[1\]"):
            a.check()
    finally:
        a.close()
        b.close()


def test_heartbeat_reports_a_rank_that_never_joins():
    store = dist.HashStore()
    a = Heartbeat(store, 0, 3, interval_s=0.05, timeout_s=0.3)
    try:
        with pytest.raises(PeerFailure, match="never joined"):
            a.wait_all_alive(0.3)
    finally:
        a.close()


def _leaving_rank_worker(rank, world):
    """Rank 1 leaves between steps (no collective in flight); rank 0 learns it from the heartbeat before its next
    collective and raises instead of blocking in it."""
    store = dist.distributed_c10d._get_default_store()
    hb = Heartbeat(store, rank, world, interval_s=0.05, timeout_s=0.5, prefix="t_leave")
    hb.wait_all_alive(10.0)
    t = torch.ones(4)
    dist.all_reduce(t)  # step 0: everyone is there
    assert float(t[0]) == world
    if rank == 1:
        hb.close()
        return "left"
    hb.check()
    time.sleep(0.8)
    try:
        hb.check()
    except PeerFailure as e:
        hb.close()
        return f"detected: {e}"
    hb.close()
    return "missed"


def test_gloo_rank_leaving_between_steps_is_detected():
    res = run_ranks(_leaving_rank_worker, 2, 29641)
    assert res[1] == "left"
    assert res[0].startswith("detected") and "[1]" in res[0], res[0]


def test_nan_policies():
    assert apply_nan_policy("ignore", float("nan"), 3) is False
    assert apply_nan_policy("skip", 1.5, 3) is False
    assert apply_nan_policy("skip", float("inf"), 3) is True
    with pytest.raises(NonFiniteLoss):
        apply_nan_policy("abort", float("nan"), 3)
    with pytest.raises(ValueError):
        apply_nan_policy("explode", float("nan"), 3)


def test_trainer_skips_update_on_non_finite_loss():
    from mintext_b200 import trainer
    from mintext_b200.models import Transformer

    cfg = MinTextConfig(dtype="float32", vocab_size=64, num_hidden_layers=1, hidden_size=32, num_attention_heads=4,
                        intermediate_size=64, seq_length=8, nan_policy="skip", learning_rate=1e-2)
    model = Transformer(cfg, rngs=0)
    state = trainer.create_train_state(model, cfg)
    tok = torch.randint(0, 64, (2, 8))
    batch = {"input_tokens": tok, "target_tokens": tok}
    state, m = trainer.train_step(state, batch, model, cfg)
    state, m = trainer.train_step(state, batch, model, cfg)
    assert not m["skipped"] and state.step == 2
    before = {n: p.detach().clone() for n, p in state.params.items()}
    with torch.no_grad():  # host-side injection: poison one weight so that the loss becomes NaN
        state.params["token_embedder"][0, 0] = float("nan")
        before["token_embedder"][0, 0] = float("nan")
    tok2 = tok.clone()
    tok2[0, 0] = 0
    state, m = trainer.train_step(state, {"input_tokens": tok2, "target_tokens": tok2}, model, cfg)
    assert m["skipped"] and state.step == 2
    for n, p in state.params.items():
        assert torch.equal(torch.nan_to_num(p), torch.nan_to_num(before[n])), n
    cfg_abort = cfg.model_copy(update={"nan_policy": "abort"})
    with pytest.raises(NonFiniteLoss):
        trainer.train_step(state, {"input_tokens": tok2, "target_tokens": tok2}, model, cfg_abort)


def test_damaged_checkpoint_is_skipped_for_the_previous_one(tmp_path):
    from mintext_b200 import trainer
    from mintext_b200.checkpoint.manager import (CheckpointCorrupt, CheckpointManager, maybe_restore_checkpoint,
                                                 save_checkpoint, wait_for_checkpoint)
    from mintext_b200.models import Transformer

    cfg = MinTextConfig(dtype="float32", vocab_size=64, num_hidden_layers=1, hidden_size=32, num_attention_heads=4,
                        intermediate_size=64, seq_length=8, checkpoint_dir=str(tmp_path), checkpoint_period=1)
    model = Transformer(cfg, rngs=0)
    state = trainer.create_train_state(model, cfg)
    mgr = CheckpointManager(str(tmp_path), save_interval_steps=1, max_to_keep=5, enable_async=False)
    tok = torch.randint(0, 64, (2, 8))
    for step in (1, 2):
        state, _ = trainer.train_step(state, {"input_tokens": tok, "target_tokens": tok}, model, cfg)
        save_checkpoint(mgr, step, state, force=True)
    wait_for_checkpoint(mgr)
    victim = max((tmp_path / "2" / "default").glob("*.bin"), key=lambda p: p.stat().st_size)
    victim.write_bytes(victim.read_bytes()[:-8])  # truncated file behind a valid commit marker
    with pytest.raises(CheckpointCorrupt):
        mgr.verify(2)
    mgr.verify(1)
    fresh = trainer.create_train_state(Transformer(cfg, rngs=1), cfg)
    fresh, start = maybe_restore_checkpoint(mgr, fresh, cfg)
    assert start == 1
    (tmp_path / "1" / "default" / "_METADATA").write_text("{not json")
    with pytest.raises(CheckpointCorrupt):
        maybe_restore_checkpoint(mgr, trainer.create_train_state(Transformer(cfg, rngs=1), cfg), cfg)


def _train_with_heartbeat_worker(rank, world):
    import os
    from pathlib import Path

    from mintext_b200.config import load_config
    from mintext_b200.train import train

    root = Path(__file__).resolve().parents[1]
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank))
    cfg = load_config([str(root / "configs" / "base.yml"), str(root / "configs" / "models" / "test-tiny.yml")],
                      dict(steps=3, seq_length=16, per_device_batch_size=2, enable_tensorboard=False,
                           enable_checkpointing=False, dtype="float32", weight_dtype="float32", kernel_backend="oracle",
                           heartbeat_interval=0.05, heartbeat_timeout=5.0, nan_policy="abort",
                           ici_fsdp_parallelism=world))
    return train(cfg)["loss"]


def test_training_loop_runs_with_heartbeats_on_gloo_ranks():
    res = run_ranks(_train_with_heartbeat_worker, 2, 29643)
    assert all(v == v for v in res.values())
