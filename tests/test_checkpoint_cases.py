"""Single-behaviour tests of the checkpoint manager and the HuggingFace key maps (after the cases of the reference's
tests/test_checkpoint.py)."""

from pathlib import Path

import pytest
import torch

from mintext_b200 import MinTextConfig, trainer
from mintext_b200.checkpoint import (create_checkpoint_manager, maybe_restore_checkpoint, restore_checkpoint,
                                     save_checkpoint, save_hf_checkpoint, wait_for_checkpoint)
from mintext_b200.checkpoint.conversion import _hf_to_mintext_key_map, _mintext_to_hf_config, _mintext_to_hf_key_map
from mintext_b200.models import Transformer


def cfg(tmp, **kw):
    base = dict(dtype="float32", vocab_size=64, num_key_value_heads=2, base_output_directory=str(tmp),
                checkpoint_period=1, max_checkpoints=3, enable_tensorboard=False, async_checkpointing=True)
    base.update(kw)
    return MinTextConfig(**base)


def make(c):
    m = Transformer(c, rngs=0)
    return m, trainer.create_train_state(m, c)


def batch(c, seed=0):
    t = torch.randint(0, c.vocab_size, (2, 16), generator=torch.Generator().manual_seed(seed))
    return {"input_tokens": t, "target_tokens": t}


@pytest.fixture
def trained(tmp_path):
    c = cfg(tmp_path)
    m, st = make(c)
    mgr = create_checkpoint_manager(c)
    for s in range(1, 4):
        st, _ = trainer.train_step(st, batch(c, s), m, c)
        save_checkpoint(mgr, s, st)
    wait_for_checkpoint(mgr)
    return c, m, st, mgr


# ---- manager -----------------------------------------------------------------------------------------------------
def test_manager_is_created_with_its_directory(tmp_path):
    c = cfg(tmp_path)
    mgr = create_checkpoint_manager(c)
    assert mgr is not None and mgr.all_steps() == [] and mgr.latest_step() is None


def test_start_without_a_manager_when_checkpointing_is_off(tmp_path):
    c = cfg(tmp_path, enable_checkpointing=False)
    m, st = make(c)
    st2, start = maybe_restore_checkpoint(None, st, c, model=m)
    assert start == 0 and st2 is st


def test_saved_steps_are_listed_in_order(trained):
    assert trained[3].all_steps() == [1, 2, 3]


def test_latest_step(trained):
    assert trained[3].latest_step() == 3


def test_restore_latest_gives_the_trained_parameters(trained):
    c, _, st, mgr = trained
    _, fresh = make(c)
    fresh, step = restore_checkpoint(mgr, fresh)
    assert step == 3
    for n, p in st.params.items():
        assert torch.equal(fresh.params[n], p), n


def test_restore_brings_back_the_optimizer_state(trained):
    c, _, st, mgr = trained
    _, fresh = make(c)
    fresh, _ = restore_checkpoint(mgr, fresh)
    assert fresh.opt_state.count == st.opt_state.count
    for n, t in st.opt_state.nu.items():
        assert torch.equal(fresh.opt_state.nu[n], t), n


def test_restore_a_named_step(trained):
    c, _, _, mgr = trained
    _, fresh = make(c)
    fresh, step = restore_checkpoint(mgr, fresh, step=2)
    assert step == 2 and fresh.step == 2


def test_restore_a_missing_step(trained):
    c, _, _, mgr = trained
    _, fresh = make(c)
    with pytest.raises(FileNotFoundError):
        restore_checkpoint(mgr, fresh, step=17)


def test_only_the_newest_checkpoints_are_kept(tmp_path):
    c = cfg(tmp_path, max_checkpoints=2)
    _, st = make(c)
    mgr = create_checkpoint_manager(c)
    for s in (1, 2, 3, 4):
        save_checkpoint(mgr, s, st)
    wait_for_checkpoint(mgr)
    assert mgr.all_steps() == [3, 4]
    assert not (Path(c.checkpoint_dir) / "1").exists()


def test_save_interval_is_respected(tmp_path):
    c = cfg(tmp_path, checkpoint_period=5)
    _, st = make(c)
    mgr = create_checkpoint_manager(c)
    assert [save_checkpoint(mgr, s, st) for s in (1, 4, 5, 6, 10)] == [False, False, True, False, True]
    wait_for_checkpoint(mgr)


def test_forced_save_ignores_the_interval(tmp_path):
    c = cfg(tmp_path, checkpoint_period=100)
    _, st = make(c)
    mgr = create_checkpoint_manager(c)
    assert save_checkpoint(mgr, 7, st, force=True)
    wait_for_checkpoint(mgr)
    assert mgr.all_steps() == [7]


def test_synchronous_saving(tmp_path):
    c = cfg(tmp_path, async_checkpointing=False)
    _, st = make(c)
    mgr = create_checkpoint_manager(c)
    save_checkpoint(mgr, 1, st)
    assert mgr.all_steps() == [1]  # committed without waiting


def test_checkpoint_tree_layout(trained):
    c = trained[0]
    step_dir = Path(c.checkpoint_dir) / "3" / "default"
    assert step_dir.is_dir() and (step_dir / "_METADATA").exists()


def test_restore_from_an_empty_directory(tmp_path):
    c = cfg(tmp_path)
    _, st = make(c)
    with pytest.raises(FileNotFoundError):
        restore_checkpoint(create_checkpoint_manager(c), st)


# ---- start-up priorities -----------------------------------------------------------------------------------------
def test_scratch_start_returns_the_initial_state(tmp_path):
    c = cfg(tmp_path)
    m, st = make(c)
    before = {n: p.clone() for n, p in st.params.items()}
    st, start = maybe_restore_checkpoint(create_checkpoint_manager(c), st, c, model=m)
    assert start == 0 and all(torch.equal(before[n], p) for n, p in st.params.items())


def test_own_directory_is_resumed(trained):
    c, _, st, _ = trained
    m2, st2 = make(c)
    st2, start = maybe_restore_checkpoint(create_checkpoint_manager(c), st2, c, model=m2)
    assert start == 3 and torch.equal(st2.params["token_embedder"], st.params["token_embedder"])


def test_external_checkpoint_full_state(trained, tmp_path):
    c = trained[0]
    c2 = cfg(tmp_path / "second", load_checkpoint=c.checkpoint_dir)
    m2, st2 = make(c2)
    st2, start = maybe_restore_checkpoint(create_checkpoint_manager(c2), st2, c2, model=m2)
    assert start == 3 and st2.opt_state.count == 3


def test_external_checkpoint_parameters_only(trained, tmp_path):
    c, _, st, _ = trained
    c2 = cfg(tmp_path / "third", load_checkpoint=c.checkpoint_dir, load_params_only=True)
    m2, st2 = make(c2)
    st2, start = maybe_restore_checkpoint(create_checkpoint_manager(c2), st2, c2, model=m2)
    assert start == 0 and st2.opt_state.count == 0
    assert torch.equal(st2.params["final_norm.scale"], st.params["final_norm.scale"])


def test_own_directory_beats_an_external_checkpoint(trained, tmp_path):
    c = trained[0]
    other = cfg(tmp_path / "other")
    mo, so = make(other)
    mgr_o = create_checkpoint_manager(other)
    save_checkpoint(mgr_o, 9, so, force=True)
    wait_for_checkpoint(mgr_o)
    c2 = c.model_copy(update={"load_checkpoint": other.checkpoint_dir})
    m2, st2 = make(c2)
    _, start = maybe_restore_checkpoint(create_checkpoint_manager(c2), st2, c2, model=m2)
    assert start == 3  # its own step 3, not the other run's step 9


def test_huggingface_directory_as_a_start(trained, tmp_path):
    c, m, st, _ = trained
    save_hf_checkpoint(m, c, str(tmp_path / "hf"))
    c2 = cfg(tmp_path / "fourth", load_hf_checkpoint=str(tmp_path / "hf"))
    m2, st2 = make(c2)
    st2, start = maybe_restore_checkpoint(create_checkpoint_manager(c2), st2, c2, model=m2)
    assert start == 0 and torch.allclose(st2.params["layers.1.attention.query.kernel"],
                                         st.params["layers.1.attention.query.kernel"])


# ---- key maps ----------------------------------------------------------------------------------------------------
FAMILIES = {
    "llama3": dict(),
    "qwen3": dict(use_qk_norm=True),
    "deepseek_v3": dict(attention_type="mla", q_lora_rank=16, kv_lora_rank=16, qk_nope_head_dim=8, qk_rope_head_dim=8,
                        v_head_dim=8, num_experts=4, num_experts_per_tok=2, moe_intermediate_size=16, n_group=2,
                        topk_group=1, first_k_dense_replace=1, n_shared_experts=1),
    "qwen3_next": dict(use_qk_norm=True, full_attention_interval=2, partial_rotary_factor=0.5, linear_key_head_dim=8,
                       linear_value_head_dim=8, linear_num_key_heads=2, linear_num_value_heads=4),
}


def _family_cfg(name):
    return MinTextConfig(dtype="float32", vocab_size=64, num_hidden_layers=2, hidden_size=32, num_attention_heads=4,
                         num_key_value_heads=2, intermediate_size=64, model_type=name, **FAMILIES[name])


@pytest.mark.parametrize("family", sorted(FAMILIES))
def test_forward_map_covers_every_parameter(family):
    c = _family_cfg(family)
    names = {n for n, _ in Transformer(c, rngs=0).named_parameters()}
    mapped = set(_mintext_to_hf_key_map(c))
    # stacked expert weights map to one HF tensor per expert and projection, so they are keyed per expert
    names = {n for n in names if ".experts." not in n}
    assert names <= mapped, sorted(names - mapped)


@pytest.mark.parametrize("family", sorted(FAMILIES))
def test_reverse_map_is_the_inverse(family):
    c = _family_cfg(family)
    fwd, rev = _mintext_to_hf_key_map(c), _hf_to_mintext_key_map(c)
    assert len(fwd) == len(rev)
    for ours, (theirs, _) in fwd.items():
        assert rev[theirs][0] == ours


def test_llama_map_names_the_layers():
    fwd = _mintext_to_hf_key_map(_family_cfg("llama3"))
    assert fwd["layers.1.mlp.down.kernel"][0] == "model.layers.1.mlp.down_proj.weight"
    assert fwd["token_embedder"][0] == "model.embed_tokens.weight" and fwd["final_norm.scale"][0] == "model.norm.weight"


def test_qwen3_map_has_the_query_key_norms():
    fwd = _mintext_to_hf_key_map(_family_cfg("qwen3"))
    assert any(v[0].endswith("self_attn.q_norm.weight") for v in fwd.values())
    assert any(v[0].endswith("self_attn.k_norm.weight") for v in fwd.values())


def test_deepseek_map_has_the_latent_projections():
    vals = {v[0] for v in _mintext_to_hf_key_map(_family_cfg("deepseek_v3")).values()}
    assert "model.layers.0.self_attn.kv_a_proj_with_mqa.weight" in vals
    assert "model.layers.1.mlp.gate.e_score_correction_bias" in vals


def test_qwen3_next_map_follows_the_layer_types():
    vals = {v[0] for v in _mintext_to_hf_key_map(_family_cfg("qwen3_next")).values()}
    assert "model.layers.0.linear_attn.in_proj_qkvz.weight" in vals   # layer 0: Gated Delta Rule
    assert "model.layers.1.self_attn.q_proj.weight" in vals           # layer 1: full attention


@pytest.mark.parametrize("family,model_type", [("llama3", "llama"), ("qwen3", "qwen3"), ("deepseek_v3", "deepseek_v3"),
                                               ("qwen3_next", "qwen3_next")])
def test_exported_hf_config_type(family, model_type):
    hf = _mintext_to_hf_config(_family_cfg(family))
    assert hf["model_type"] == model_type and hf["hidden_size"] == 32 and hf["num_hidden_layers"] == 2


def test_exported_hf_config_basic_fields():
    hf = _mintext_to_hf_config(_family_cfg("llama3"))
    assert hf["vocab_size"] == 64 and hf["num_attention_heads"] == 4 and hf["num_key_value_heads"] == 2
    assert hf["intermediate_size"] == 64 and "rms_norm_eps" in hf and "rope_theta" in hf
