"""Single-behaviour tests of the config model and its loader (defaults, derived fields, validators, YAML chains,
command-line and environment overrides), after the cases of the reference's tests/test_config.py."""

from pathlib import Path

import pytest
import yaml

from mintext_b200.config import MinTextConfig, load_config, parse_cli_overrides, print_help_config

CONFIGS = Path(__file__).resolve().parents[1] / "configs"


def _write(tmp_path, name, data):
    p = tmp_path / name
    p.write_text(yaml.safe_dump(data))
    return p


# ---- defaults and derived fields ---------------------------------------------------------------------------------
def test_default_config_is_valid():
    c = MinTextConfig()
    assert c.num_hidden_layers >= 1 and c.vocab_size >= 1 and c.steps >= 0


def test_head_dim_is_derived_from_width_and_heads():
    assert MinTextConfig(hidden_size=256, num_attention_heads=8).head_dim == 32


def test_kv_heads_default_to_query_heads():
    assert MinTextConfig(num_attention_heads=6, hidden_size=96).num_key_value_heads == 6


def test_explicit_head_dim_is_kept():
    assert MinTextConfig(hidden_size=256, num_attention_heads=8, head_dim=48).head_dim == 48


def test_explicit_kv_heads_are_kept():
    assert MinTextConfig(num_attention_heads=8, hidden_size=256, num_key_value_heads=2).num_key_value_heads == 2


def test_default_logical_axis_rules_start_with_the_batch_rule():
    assert tuple(MinTextConfig().logical_axis_rules[0]) == ("batch", "data")


def test_default_output_directories_hang_off_the_run_name():
    c = MinTextConfig(run_name="exp7", base_output_directory="/tmp/out")
    assert c.checkpoint_dir == "/tmp/out/exp7/checkpoints"
    assert c.tensorboard_dir == "/tmp/out/exp7/tensorboard" and c.log_dir == "/tmp/out/exp7/logs"


def test_layer_types_default_to_full_attention():
    assert MinTextConfig(num_hidden_layers=3).layer_types == ["full_attention"] * 3


def test_qwen3_next_layer_types_follow_the_interval():
    c = MinTextConfig(model_type="qwen3_next", num_hidden_layers=4, full_attention_interval=2)
    assert c.layer_types == ["linear_attention", "full_attention", "linear_attention", "full_attention"]


def test_mla_query_key_head_dim_is_the_sum_of_its_parts():
    assert MinTextConfig(qk_nope_head_dim=96, qk_rope_head_dim=32).qk_head_dim == 128


def test_dtype_helpers():
    import torch

    c = MinTextConfig(dtype="float32", weight_dtype="float32")
    assert c.torch_dtype == torch.float32 and c.torch_weight_dtype == torch.float32


# ---- validators --------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("field", ["num_hidden_layers", "hidden_size", "num_attention_heads", "vocab_size",
                                   "per_device_batch_size"])
@pytest.mark.parametrize("value", [0, -3])
def test_sizes_must_be_positive(field, value):
    with pytest.raises(ValueError):
        MinTextConfig(**{field: value})


def test_steps_may_be_zero_but_not_negative():
    assert MinTextConfig(steps=0).steps == 0
    with pytest.raises(ValueError):
        MinTextConfig(steps=-1)


def test_vocab_tiles_must_divide_the_token_count():
    with pytest.raises(ValueError, match="num_vocab_tiles"):
        MinTextConfig(per_device_batch_size=1, seq_length=10, num_vocab_tiles=3)
    assert MinTextConfig(per_device_batch_size=2, seq_length=8, num_vocab_tiles=4).num_vocab_tiles == 4


def test_two_checkpoint_sources_are_rejected():
    with pytest.raises(ValueError, match="mutually exclusive"):
        MinTextConfig(load_checkpoint="/a", load_hf_checkpoint="/b")


def test_params_only_needs_a_checkpoint():
    with pytest.raises(ValueError, match="load_checkpoint"):
        MinTextConfig(load_params_only=True)


def test_unknown_enum_value_is_rejected():
    with pytest.raises(ValueError):
        MinTextConfig(optimizer="sgd")
    with pytest.raises(ValueError):
        MinTextConfig(remat_policy="sometimes")


# ---- immutability ------------------------------------------------------------------------------------------------
def test_fields_cannot_be_assigned():
    c = MinTextConfig()
    with pytest.raises(Exception):
        c.learning_rate = 1.0


def test_fields_cannot_be_deleted():
    c = MinTextConfig()
    with pytest.raises(Exception):
        del c.learning_rate


def test_model_copy_gives_a_changed_copy():
    c = MinTextConfig(steps=3)
    d = c.model_copy(update={"steps": 9})
    assert (c.steps, d.steps) == (3, 9)


# ---- YAML --------------------------------------------------------------------------------------------------------
def test_base_yml_loads():
    assert load_config(CONFIGS / "base.yml").num_hidden_layers >= 1


def test_test_tiny_inherits_from_base():
    c = load_config(CONFIGS / "models" / "test-tiny.yml")
    assert c.hidden_size == 128 and c.vocab_size == 256 and c.num_hidden_layers == 2
    assert c.learning_rate == load_config(CONFIGS / "base.yml").learning_rate  # not set by the child


def test_llama3_8b_preset():
    c = load_config(CONFIGS / "models" / "meta-llama-3-8b.yml")
    assert (c.num_hidden_layers, c.hidden_size, c.num_attention_heads, c.num_key_value_heads) == (32, 4096, 32, 8)
    assert c.intermediate_size == 14336 and c.vocab_size == 128256


def test_deepseek_preset_is_mla_with_experts():
    c = load_config(CONFIGS / "models" / "deepseek-v3.yml")
    assert c.attention_type == "mla" and c.num_experts == 256 and c.n_shared_experts == 1 and c.first_k_dense_replace == 3


def test_overrides_are_applied(tmp_path):
    p = _write(tmp_path, "c.yml", {"steps": 3})
    assert load_config(p, {"hidden_size": 64}).hidden_size == 64


def test_overrides_beat_the_yaml(tmp_path):
    p = _write(tmp_path, "c.yml", {"steps": 3})
    assert load_config(p, {"steps": 8}).steps == 8


def test_enum_fields_from_yaml(tmp_path):
    p = _write(tmp_path, "c.yml", {"optimizer": "muon", "lr_schedule": "wsd", "remat_policy": "full"})
    c = load_config(p)
    assert (c.optimizer, c.lr_schedule, c.remat_policy) == ("muon", "wsd", "full")


def test_missing_yaml_file():
    with pytest.raises(FileNotFoundError):
        load_config("/no/such/config.yml")


def test_base_chain_of_three(tmp_path):
    _write(tmp_path, "a.yml", {"hidden_size": 64, "steps": 1, "vocab_size": 99})
    _write(tmp_path, "b.yml", {"base_config": "a.yml", "steps": 2})
    c = load_config(_write(tmp_path, "c.yml", {"base_config": "b.yml", "vocab_size": 77}))
    assert (c.hidden_size, c.steps, c.vocab_size) == (64, 2, 77)


def test_base_chain_cycle_is_detected(tmp_path):
    _write(tmp_path, "a.yml", {"base_config": "b.yml"})
    p = _write(tmp_path, "b.yml", {"base_config": "a.yml"})
    with pytest.raises(ValueError):
        load_config(p)


def test_unknown_yaml_key_is_ignored_like_any_unknown_constructor_argument(tmp_path):
    p = _write(tmp_path, "c.yml", {"some_key_of_another_tool": 64, "steps": 3})
    assert load_config(p).steps == 3


# ---- unknown keys ------------------------------------------------------------------------------------------------
def test_typo_gets_a_suggestion(tmp_path):
    p = _write(tmp_path, "c.yml", {})
    with pytest.raises(ValueError, match="did you mean 'num_hidden_layers'"):
        load_config(p, {"num_hiden_layers": 3})


def test_unrelated_key_gets_no_suggestion(tmp_path):
    p = _write(tmp_path, "c.yml", {})
    with pytest.raises(ValueError) as info:
        load_config(p, {"qqqqzzzz": 1})
    assert "did you mean" not in str(info.value)


def test_several_unknown_keys_are_all_listed(tmp_path):
    p = _write(tmp_path, "c.yml", {})
    with pytest.raises(ValueError) as info:
        load_config(p, {"stepz": 1, "learning_rat": 2.0})
    assert "stepz" in str(info.value) and "learning_rat" in str(info.value)


def test_known_keys_pass(tmp_path):
    p = _write(tmp_path, "c.yml", {})
    c = load_config(p, {"steps": 4, "learning_rate": 0.5, "run_name": "r"})
    assert (c.steps, c.learning_rate, c.run_name) == (4, 0.5, "r")


# ---- environment -------------------------------------------------------------------------------------------------
def test_env_int(tmp_path, monkeypatch):
    monkeypatch.setenv("MINTEXT_STEPS", "42")
    assert load_config(_write(tmp_path, "c.yml", {"steps": 1})).steps == 42


def test_env_float(tmp_path, monkeypatch):
    monkeypatch.setenv("MINTEXT_LEARNING_RATE", "2.5e-4")
    assert load_config(_write(tmp_path, "c.yml", {"learning_rate": 0.1})).learning_rate == 2.5e-4


def test_env_string(tmp_path, monkeypatch):
    monkeypatch.setenv("MINTEXT_RUN_NAME", "from_env")
    assert load_config(_write(tmp_path, "c.yml", {"run_name": "yaml"})).run_name == "from_env"


@pytest.mark.parametrize("raw,expected", [("true", True), ("1", True), ("yes", True), ("false", False), ("0", False),
                                          ("No", False)])
def test_env_bool_spellings(tmp_path, monkeypatch, raw, expected):
    monkeypatch.setenv("MINTEXT_TIE_WORD_EMBEDDINGS", raw)
    c = load_config(_write(tmp_path, "c.yml", {"tie_word_embeddings": not expected}))
    assert c.tie_word_embeddings is expected


def test_env_bool_garbage(tmp_path, monkeypatch):
    monkeypatch.setenv("MINTEXT_TIE_WORD_EMBEDDINGS", "perhaps")
    with pytest.raises(ValueError, match="Cannot parse"):
        load_config(_write(tmp_path, "c.yml", {"tie_word_embeddings": True}))


def test_env_and_cli_for_the_same_key_is_an_error(tmp_path, monkeypatch):
    monkeypatch.setenv("MINTEXT_STEPS", "5")
    with pytest.raises(ValueError, match="both CLI and environment"):
        load_config(_write(tmp_path, "c.yml", {"steps": 1}), {"steps": 6})


def test_env_for_other_keys_does_not_clash_with_cli(tmp_path, monkeypatch):
    monkeypatch.setenv("MINTEXT_STEPS", "5")
    c = load_config(_write(tmp_path, "c.yml", {"steps": 1}), {"hidden_size": 64})
    assert (c.steps, c.hidden_size) == (5, 64)


def test_unrelated_environment_is_ignored(tmp_path, monkeypatch):
    monkeypatch.setenv("MINTEXT_NOT_A_FIELD", "1")
    monkeypatch.setenv("OTHER_STEPS", "9")
    assert load_config(_write(tmp_path, "c.yml", {"steps": 2})).steps == 2


# ---- command line ------------------------------------------------------------------------------------------------
def test_cli_int_float_bool_string():
    o = parse_cli_overrides(["steps=5", "learning_rate=0.25", "tie_word_embeddings=false", "run_name=abc"])
    assert o == {"steps": 5, "learning_rate": 0.25, "tie_word_embeddings": False, "run_name": "abc"}


def test_cli_scientific_notation_is_a_float():
    assert parse_cli_overrides(["learning_rate=3e-4"])["learning_rate"] == 3e-4


def test_cli_list_value():
    assert parse_cli_overrides(["moe_down_tiling=[256,64,256]"])["moe_down_tiling"] == [256, 64, 256]


def test_cli_value_with_equals_sign():
    assert parse_cli_overrides(["run_name=a=b"])["run_name"] == "a=b"


def test_cli_leading_dashes_are_accepted():
    assert parse_cli_overrides(["--steps=3"]) == {"steps": 3}


def test_cli_token_without_equals():
    with pytest.raises(ValueError, match="key=value"):
        parse_cli_overrides(["steps"])


def test_cli_int_override_through_load_config(tmp_path):
    p = _write(tmp_path, "c.yml", {"steps": 1})
    assert load_config(p, parse_cli_overrides(["steps=12"])).steps == 12


def test_help_lists_every_field(capsys):
    print_help_config()
    out = capsys.readouterr().out
    for name in ("learning_rate", "ici_fsdp_parallelism", "fsdp_shard_params", "remat_policy"):
        assert name in out
    assert f"Total: {len(MinTextConfig.model_fields)}" in out


def test_exponent_literals_without_a_dot_load_as_numbers(tmp_path):
    """PyYAML reads ``1e-5`` (no dot) as a string; the reference's config files are written that way."""
    f = tmp_path / "c.yml"
    f.write_text("rms_norm_eps: 1e-5\nlearning_rate: 3e-4\nadam_eps: 1e-8\nrope_theta: 500000.0\n")
    c = load_config(f)
    assert c.rms_norm_eps == 1e-5 and c.learning_rate == 3e-4 and c.adam_eps == 1e-8
    assert isinstance(c.rms_norm_eps, float)
