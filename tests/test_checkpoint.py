"""Checkpoint manager semantics, HF key maps, safetensors round-trip and logit parity with ``transformers``."""

import json
from pathlib import Path

import pytest
import torch

from mintext_b200 import MinTextConfig, trainer
from mintext_b200.checkpoint import (create_checkpoint_manager, load_hf_checkpoint, maybe_restore_checkpoint,
                                     restore_checkpoint, save_checkpoint, save_hf_checkpoint, wait_for_checkpoint)
from mintext_b200.checkpoint.conversion import (_hf_to_mintext_key_map, _mintext_to_hf_config, _mintext_to_hf_key_map,
                                                key_table)
from mintext_b200.models import Transformer


def cfg(tmp, **kw):
    base = dict(dtype="float32", vocab_size=64, num_key_value_heads=2, base_output_directory=str(tmp),
                checkpoint_period=1, max_checkpoints=2, enable_tensorboard=False, async_checkpointing=True)
    base.update(kw)
    return MinTextConfig(**base)


def make_state(c):
    m = Transformer(c, rngs=0)
    return m, trainer.create_train_state(m, c)


def batch(c, seed=0):
    g = torch.Generator().manual_seed(seed)
    t = torch.randint(0, c.vocab_size, (2, 16), generator=g)
    return {"input_tokens": t, "target_tokens": t}


def snapshot(state):
    return {n: p.detach().clone() for n, p in state.params.items()}


def test_save_restore_roundtrip_latest_and_retention(tmp_path):
    c = cfg(tmp_path)
    m, st = make_state(c)
    mgr = create_checkpoint_manager(c)
    for s in range(1, 5):
        st, _ = trainer.train_step(st, batch(c, s), m, c)
        assert save_checkpoint(mgr, s, st)
    wait_for_checkpoint(mgr)
    assert mgr.all_steps() == [3, 4] and mgr.latest_step() == 4
    want = snapshot(st)
    want_mu = {n: t.clone() for n, t in st.opt_state.mu.items()}
    m2, st2 = make_state(c)
    st2, step = restore_checkpoint(mgr, st2)
    assert step == 4 and st2.step == 4 and st2.opt_state.count == st.opt_state.count
    for n in want:
        assert torch.equal(st2.params[n], want[n])
    for n in want_mu:
        assert torch.equal(st2.opt_state.mu[n], want_mu[n])
    st3 = make_state(c)[1]
    assert restore_checkpoint(mgr, st3, step=3)[1] == 3


def test_interval_force_and_missing(tmp_path):
    c = cfg(tmp_path, checkpoint_period=10)
    m, st = make_state(c)
    mgr = create_checkpoint_manager(c)
    assert not save_checkpoint(mgr, 3, st)
    assert save_checkpoint(mgr, 3, st, force=True)
    assert save_checkpoint(mgr, 10, st)
    wait_for_checkpoint(mgr)
    assert mgr.all_steps() == [3, 10]
    empty = create_checkpoint_manager(cfg(tmp_path / "other"))
    with pytest.raises(FileNotFoundError):
        restore_checkpoint(empty, st)


def test_uncommitted_step_is_ignored(tmp_path):
    c = cfg(tmp_path)
    m, st = make_state(c)
    mgr = create_checkpoint_manager(c)
    save_checkpoint(mgr, 1, st)
    wait_for_checkpoint(mgr)
    broken = Path(c.checkpoint_dir) / "2" / "default"
    broken.mkdir(parents=True)
    (broken / "_METADATA").write_text("{}")  # files but no commit marker: a crash mid-save
    assert mgr.latest_step() == 1


def test_maybe_restore_priorities(tmp_path):
    # (4) scratch
    c = cfg(tmp_path / "run1")
    m, st = make_state(c)
    mgr = create_checkpoint_manager(c)
    st, start = maybe_restore_checkpoint(mgr, st, c, model=m)
    assert start == 0
    for s in range(1, 4):
        st, _ = trainer.train_step(st, batch(c, s), m, c)
    save_checkpoint(mgr, 3, st, force=True)
    wait_for_checkpoint(mgr)
    trained = snapshot(st)
    # (1) own directory wins
    m1, st1 = make_state(c)
    st1, start = maybe_restore_checkpoint(create_checkpoint_manager(c), st1, c, model=m1)
    assert start == 3 and torch.equal(st1.params["token_embedder"], trained["token_embedder"])
    # (2) load_checkpoint: full state, then parameters only
    c2 = cfg(tmp_path / "run2", load_checkpoint=c.checkpoint_dir)
    m2, st2 = make_state(c2)
    st2, start = maybe_restore_checkpoint(create_checkpoint_manager(c2), st2, c2, model=m2)
    assert start == 3 and st2.opt_state.count == 3
    c3 = cfg(tmp_path / "run3", load_checkpoint=c.checkpoint_dir, load_params_only=True)
    m3, st3 = make_state(c3)
    st3, start = maybe_restore_checkpoint(create_checkpoint_manager(c3), st3, c3, model=m3)
    assert start == 0 and st3.step == 0 and st3.opt_state.count == 0
    assert torch.equal(st3.params["token_embedder"], trained["token_embedder"])
    assert float(st3.opt_state.mu["token_embedder"].abs().sum()) == 0.0
    # (3) HF directory
    hf_dir = tmp_path / "hf"
    save_hf_checkpoint(m, c, str(hf_dir))
    c4 = cfg(tmp_path / "run4", load_hf_checkpoint=str(hf_dir))
    m4, st4 = make_state(c4)
    st4, start = maybe_restore_checkpoint(create_checkpoint_manager(c4), st4, c4, model=m4)
    assert start == 0 and torch.allclose(st4.params["layers.0.mlp.gate.kernel"], trained["layers.0.mlp.gate.kernel"])


def test_restart_continues_identically(tmp_path):
    """run(0->6) == run(0->3) + restart + run(3->6)."""
    c = cfg(tmp_path / "a", steps=6)
    m, st = make_state(c)
    for s in range(6):
        st, met = trainer.train_step(st, batch(c, s), m, c)
    full = float(met["loss"])
    c2 = cfg(tmp_path / "b", steps=6)
    m2, st2 = make_state(c2)
    mgr = create_checkpoint_manager(c2)
    for s in range(3):
        st2, _ = trainer.train_step(st2, batch(c2, s), m2, c2)
    save_checkpoint(mgr, 3, st2, force=True)
    wait_for_checkpoint(mgr)
    m3, st3 = make_state(c2)
    st3, start = maybe_restore_checkpoint(create_checkpoint_manager(c2), st3, c2, model=m3)
    for s in range(start, 6):
        st3, met3 = trainer.train_step(st3, batch(c2, s), m3, c2)
    assert float(met3["loss"]) == pytest.approx(full, rel=1e-6)


# ------------------------------------------------------------------ HF conversion
def test_key_map_roundtrip_counts():
    c = MinTextConfig(num_hidden_layers=3, num_key_value_heads=2)
    fwd, back = _hf_to_mintext_key_map(c), _mintext_to_hf_key_map(c)
    assert len(fwd) == len(back) == 3 + 3 * 9
    for hf, (mt, _) in fwd.items():
        assert back[mt][0] == hf


@pytest.mark.parametrize("code,shape", [("T", (6, 4)), ("qkv:2,3", (6, 5)), ("out:2,3", (5, 6)), ("norm1", (7,))])
def test_transforms_invert_exactly(code, shape):
    from mintext_b200.checkpoint.conversion import _apply

    t = torch.randn(shape)
    back = _apply(code, _apply(code, t), inverse=True)
    assert torch.allclose(back, t, atol=1e-6) if code == "norm1" else torch.equal(back, t)


def test_family_specific_keys():
    ds = MinTextConfig(model_type="deepseek_v3", attention_type="mla", q_lora_rank=8, num_hidden_layers=2, num_experts=4,
                       first_k_dense_replace=1, n_group=2, topk_group=1, num_experts_per_tok=2)
    keys = {hf for hf, _, _ in key_table(ds)}
    assert "model.layers.0.self_attn.kv_a_proj_with_mqa.weight" in keys and "model.layers.0.mlp.gate_proj.weight" in keys
    assert "model.layers.1.mlp.gate.e_score_correction_bias" in keys and "model.layers.1.mlp.shared_experts.up_proj.weight" in keys
    qn = MinTextConfig(model_type="qwen3_next", num_hidden_layers=2, full_attention_interval=2, use_qk_norm=True)
    rows = {hf: code for hf, _, code in key_table(qn)}
    assert rows["model.layers.0.linear_attn.norm.weight"] == "id" and rows["model.layers.1.self_attn.q_norm.weight"] == "norm1"
    assert rows["model.layers.0.input_layernorm.weight"] == "norm1" and "model.layers.0.linear_attn.A_log" in rows
    g = MinTextConfig(model_type="gemma3", use_post_ffw_norm=True, num_hidden_layers=1)
    assert "model.layers.0.pre_feedforward_layernorm.weight" in {hf for hf, _, _ in key_table(g)}


def test_hf_config_export():
    c = MinTextConfig(rope_type="llama3", rope_scaling_factor=8.0, rope_original_max_position_embeddings=64)
    h = _mintext_to_hf_config(c)
    assert h["architectures"] == ["LlamaForCausalLM"] and h["rope_scaling"]["rope_type"] == "llama3"
    assert _mintext_to_hf_config(MinTextConfig(model_type="gemma3"))["model_type"] == "gemma3_text"


def test_safetensors_export_import_equality(tmp_path):
    c = MinTextConfig(dtype="float32", vocab_size=64, num_key_value_heads=2, model_type="deepseek_v3", attention_type="mla",
                      q_lora_rank=8, kv_lora_rank=8, qk_nope_head_dim=8, qk_rope_head_dim=4, v_head_dim=8,
                      num_experts=4, num_experts_per_tok=2, moe_intermediate_size=16, n_group=2, topk_group=1,
                      first_k_dense_replace=1)
    a = Transformer(c, rngs=0)
    a.layers[1].mlp.router.e_score_correction_bias.data.normal_()
    save_hf_checkpoint(a, c, str(tmp_path))
    assert json.loads((tmp_path / "config.json").read_text())["n_routed_experts"] == 4
    b = Transformer(c, rngs=1)
    load_hf_checkpoint(str(tmp_path), c, b)
    for (n, p), (_, q) in zip(a.named_parameters(), b.named_parameters()):
        assert torch.equal(p, q), n


# ------------------------------------------------------------------ logit parity with transformers
def _parity(c, hf_cls_name, tmp_path, atol=1e-3):
    tr = pytest.importorskip("transformers")
    if not hasattr(tr, hf_cls_name):
        pytest.skip(f"transformers has no {hf_cls_name}")
    ours = Transformer(c, rngs=0)
    with torch.no_grad():  # give norms non-trivial scales so the +1 conventions are exercised
        for n, p in ours.named_parameters():
            if n.endswith("scale"):
                p.add_(0.1 * torch.randn_like(p))
    save_hf_checkpoint(ours, c, str(tmp_path))
    hf = getattr(tr, hf_cls_name).from_pretrained(str(tmp_path), torch_dtype=torch.float32, attn_implementation="eager")
    hf.eval()
    tok = torch.randint(0, c.vocab_size, (2, 24), generator=torch.Generator().manual_seed(0))
    with torch.no_grad():
        ref = hf(tok).logits
        got, _ = ours(tok, torch.arange(24)[None].expand(2, -1))
    cos = torch.nn.functional.cosine_similarity(got.reshape(-1), ref.reshape(-1), dim=0)
    assert cos > 0.999, cos
    assert torch.allclose(got, ref, atol=atol), (got - ref).abs().max()
    # and the other direction: HF weights -> our model
    hf.save_pretrained(str(tmp_path / "back"), safe_serialization=True)
    again = Transformer(c, rngs=5)
    load_hf_checkpoint(str(tmp_path / "back"), c, again)
    with torch.no_grad():
        got2, _ = again(tok, torch.arange(24)[None].expand(2, -1))
    assert torch.allclose(got2, ref, atol=atol)


def _base(**kw):
    base = dict(dtype="float32", vocab_size=96, num_hidden_layers=2, hidden_size=64, num_attention_heads=4,
                num_key_value_heads=2, intermediate_size=128, seq_length=64)
    base.update(kw)
    return MinTextConfig(**base)


def test_parity_llama(tmp_path):
    _parity(_base(rope_type="llama3", rope_scaling_factor=4.0, rope_original_max_position_embeddings=16,
                  rope_theta=10000.0), "LlamaForCausalLM", tmp_path)


def test_parity_qwen3(tmp_path):
    _parity(_base(model_type="qwen3", use_qk_norm=True, head_dim=32, tie_word_embeddings=True), "Qwen3ForCausalLM", tmp_path)


def test_parity_deepseek_v3(tmp_path):
    _parity(_base(model_type="deepseek_v3", attention_type="mla", q_lora_rank=16, kv_lora_rank=16, qk_nope_head_dim=16,
                  qk_rope_head_dim=8, v_head_dim=16, num_experts=8, num_experts_per_tok=2, moe_intermediate_size=32,
                  n_group=4, topk_group=2, first_k_dense_replace=1, n_shared_experts=1, rope_interleave=True),
            "DeepseekV3ForCausalLM", tmp_path)


def test_parity_qwen3_next(tmp_path):
    _parity(_base(model_type="qwen3_next", use_qk_norm=True, head_dim=32, full_attention_interval=2,
                  partial_rotary_factor=0.25, linear_key_head_dim=16, linear_value_head_dim=16, linear_num_key_heads=2,
                  linear_num_value_heads=4, num_experts=4, num_experts_per_tok=2, moe_intermediate_size=32, n_group=1,
                  topk_group=1, first_k_dense_replace=0, n_shared_experts=1, routed_scaling_factor=1.0,
                  router_type="softmax_topk", shared_expert_gate=True),
            "Qwen3NextForCausalLM", tmp_path, atol=2e-3)


def test_parity_gemma3(tmp_path):
    _parity(_base(model_type="gemma3", use_qk_norm=True, head_dim=16, query_pre_attn_scalar=16.0,
                  attn_logit_softcapping=None, final_logit_softcapping=30.0, use_post_ffw_norm=True,
                  scale_embeddings=True, sliding_window=8, sliding_window_pattern=2,
                  hidden_activation="gelu_pytorch_tanh", tie_word_embeddings=True, rope_theta=1e6, rope_local_theta=1e4,
                  rms_norm_eps=1e-6), "Gemma3ForCausalLM", tmp_path, atol=2e-3)


# ------------------------------------------------------------------ sharded entries and failing writers
class _ShardedState:
    """Stand-in for an engine whose ``w`` is column-split over ``count`` tensor-parallel ranks and whose ``e`` is
    split along dim 0 (experts)."""

    FULL_W = torch.arange(6 * 8, dtype=torch.float32).reshape(6, 8)
    FULL_E = torch.arange(4 * 3 * 2, dtype=torch.float32).reshape(4, 3, 2)

    def __init__(self, index, count, rank):
        self.index, self.count, self.rank = index, count, rank
        self.w = torch.zeros(6, 8 // count)
        self.e = torch.zeros(4 // count, 3, 2)

    def fill(self):
        self.w = self.FULL_W.chunk(self.count, 1)[self.index].contiguous()
        self.e = self.FULL_E.chunk(self.count, 0)[self.index].contiguous()

    def checkpoint_tree(self):
        def meta(dim):
            return {"writer_rank": self.rank, "shard": (dim, self.index, self.count),
                    "suffix": f".shard{self.index}of{self.count}"}
        return {"step": 1, "params/w": {"tensor": self.w, **meta(1)}, "params/e": {"tensor": self.e, **meta(0)}}

    def load_checkpoint_tree(self, read):
        self.w = read("params/w", shard=(1, self.index, self.count))
        self.e = read("params/e", shard=(0, self.index, self.count))


def _save_two_shards(rank, world, directory):
    from mintext_b200.checkpoint.manager import CheckpointManager

    st = _ShardedState(rank, world, rank)
    st.fill()
    m = CheckpointManager(directory, enable_async=False)
    assert m.save(1, st, force=True)
    back = _ShardedState(rank, world, rank)
    m.restore(1, back)
    return bool(torch.equal(back.w, st.w) and torch.equal(back.e, st.e))


def test_tensor_parallel_shards_restore_under_another_degree(tmp_path):
    """Saved by two ranks split along their shard dimensions; restored whole (degree 1) and in four shards."""
    import functools

    from mintext_b200.checkpoint.manager import CheckpointManager
    from tests.test_sharding import run_ranks

    out = run_ranks(functools.partial(_save_two_shards, directory=str(tmp_path)), 2, 29641)
    assert out == {0: True, 1: True}
    m = CheckpointManager(str(tmp_path), read_only=True)
    one = _ShardedState(0, 1, 0)
    m.restore(1, one)
    assert torch.equal(one.w, _ShardedState.FULL_W) and torch.equal(one.e, _ShardedState.FULL_E)
    for i in range(4):
        q = _ShardedState(i, 4, 0)
        m.restore(1, q)
        assert torch.equal(q.w, _ShardedState.FULL_W.chunk(4, 1)[i]) and torch.equal(q.e, _ShardedState.FULL_E[i:i + 1])
    meta = json.loads((tmp_path / "1" / "default" / "_METADATA").read_text())
    assert [c["shard"] for c in meta["params/w"]["shards"]] == [[1, 0, 2], [1, 1, 2]]


def test_failed_background_write_commits_nothing(tmp_path, monkeypatch):
    from mintext_b200.checkpoint import manager as mgr_mod

    class _FailingWriter:
        failed = False

        def submit(self, path, host):
            pass

        def wait(self):
            if not self.failed:  # like the real writers: an error is reported once, then cleared
                self.failed = True
                raise OSError("disk full")

    c = MinTextConfig(num_hidden_layers=1, hidden_size=32, num_attention_heads=2, intermediate_size=64, vocab_size=64,
                      seq_length=8, dtype="float32", checkpoint_dir=str(tmp_path), checkpoint_period=1,
                      async_checkpointing=True, enable_tensorboard=False)
    state = trainer.create_train_state(Transformer(c, rngs=0), c)
    m = create_checkpoint_manager(c)
    monkeypatch.setattr(mgr_mod, "_make_writer", lambda: _FailingWriter())
    assert m.save(1, state)
    with pytest.raises(RuntimeError, match="nothing was committed"):
        m.wait_until_finished()
    assert m.all_steps() == [] and not (tmp_path / "1").exists()
    m.wait_until_finished()          # the failed save is gone: nothing left to commit, no error
    assert m.all_steps() == []
    m._writer = None
    monkeypatch.undo()
    assert m.save(1, state) and (m.wait_until_finished() or True)
    assert m.all_steps() == [1]
