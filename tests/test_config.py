"""Config model, YAML inheritance, CLI / environment overrides (mirrors the reference's tests/test_config.py)."""

import pytest
import yaml

from mintext_b200.config import MinTextConfig, load_config, parse_cli_overrides, print_help_config


def test_defaults_and_derived_fields():
    c = MinTextConfig()
    assert c.head_dim == 32 and c.num_key_value_heads == 4
    assert c.layer_types == ["full_attention", "full_attention"]
    assert c.checkpoint_dir.endswith("default/checkpoints")
    assert c.tensorboard_dir.endswith("default/tensorboard") and c.log_dir.endswith("default/logs")
    assert c.logical_axis_rules[0] == ("batch", "data")
    assert c.qk_head_dim == 192
    assert c.linear_num_key_heads == 4 and c.linear_num_value_heads == 4


def test_explicit_values_win_over_derivation():
    c = MinTextConfig(hidden_size=256, num_attention_heads=8, head_dim=64, num_key_value_heads=2)
    assert c.head_dim == 64 and c.num_key_value_heads == 2


@pytest.mark.parametrize("field,value,msg", [
    ("num_hidden_layers", 0, "num_hidden_layers must be >= 1"), ("hidden_size", 0, "hidden_size must be >= 1"),
    ("num_attention_heads", 0, "num_attention_heads must be >= 1"), ("vocab_size", 0, "vocab_size must be >= 1"),
    ("steps", -1, "steps must be >= 0"), ("per_device_batch_size", 0, "per_device_batch_size must be >= 1")])
def test_validators(field, value, msg):
    with pytest.raises(ValueError, match=msg):
        MinTextConfig(**{field: value})


def test_vocab_tiling_and_checkpoint_source_checks():
    with pytest.raises(ValueError, match="divisible by num_vocab_tiles"):
        MinTextConfig(per_device_batch_size=1, seq_length=10, num_vocab_tiles=3)
    with pytest.raises(ValueError, match="mutually exclusive"):
        MinTextConfig(load_checkpoint="a", load_hf_checkpoint="b")
    with pytest.raises(ValueError, match="requires `load_checkpoint`"):
        MinTextConfig(load_params_only=True)


def test_frozen_and_enum_values():
    c = MinTextConfig()
    with pytest.raises(Exception):
        c.steps = 5
    assert c.dtype == "bfloat16" and c.optimizer == "adamw"
    assert MinTextConfig(rope_type="llama3_1").rope_type == "llama3"
    import torch

    assert c.torch_dtype == torch.bfloat16 and c.torch_weight_dtype == torch.float32


def test_unknown_constructor_kwargs_are_ignored():
    assert MinTextConfig(rope_original_seq_length=8192).seq_length == 128


def _write(tmp_path, name, data):
    p = tmp_path / name
    p.write_text(yaml.safe_dump(data))
    return p


def test_yaml_inheritance_and_overrides(tmp_path):
    _write(tmp_path, "base.yml", {"hidden_size": 64, "steps": 3, "learning_rate": 0.01})
    child = _write(tmp_path, "child.yml", {"base_config": "base.yml", "steps": 7})
    c = load_config(child)
    assert (c.hidden_size, c.steps, c.learning_rate) == (64, 7, 0.01)
    c = load_config(child, {"steps": 9, "hidden_size": 32})
    assert (c.hidden_size, c.steps) == (32, 9)


def test_multiple_config_files_merge_left_to_right(tmp_path):
    a = _write(tmp_path, "a.yml", {"steps": 3, "hidden_size": 64})
    b = _write(tmp_path, "b.yml", {"steps": 5})
    c = load_config([a, b])
    assert (c.steps, c.hidden_size) == (5, 64)


def test_unknown_override_key_suggests_fix(tmp_path):
    p = _write(tmp_path, "c.yml", {})
    with pytest.raises(ValueError, match="did you mean 'learning_rate'"):
        load_config(p, {"learning_rat": 1.0})
    with pytest.raises(ValueError, match="Unknown config key"):
        load_config(p, {"zzzzqqq": 1})


def test_env_overrides_typed(tmp_path, monkeypatch):
    p = _write(tmp_path, "c.yml", {"steps": 3, "learning_rate": 0.1, "run_name": "x", "tie_word_embeddings": False})
    monkeypatch.setenv("MINTEXT_STEPS", "11")
    monkeypatch.setenv("MINTEXT_LEARNING_RATE", "3e-4")
    monkeypatch.setenv("MINTEXT_RUN_NAME", "envrun")
    monkeypatch.setenv("MINTEXT_TIE_WORD_EMBEDDINGS", "true")
    c = load_config(p)
    assert (c.steps, c.learning_rate, c.run_name, c.tie_word_embeddings) == (11, 3e-4, "envrun", True)
    with pytest.raises(ValueError, match="both CLI and environment"):
        load_config(p, {"steps": 5})
    monkeypatch.setenv("MINTEXT_TIE_WORD_EMBEDDINGS", "maybe")
    monkeypatch.delenv("MINTEXT_STEPS")
    with pytest.raises(ValueError, match="Cannot parse"):
        load_config(p)


def test_cli_override_parsing():
    o = parse_cli_overrides(["steps=5", "learning_rate=1e-4", "tie_word_embeddings=true", "run_name=abc",
                             "moe_gate_up_tiling=[128,128,64]", "data_split=99,1,0"])
    assert o == {"steps": 5, "learning_rate": 1e-4, "tie_word_embeddings": True, "run_name": "abc",
                 "moe_gate_up_tiling": [128, 128, 64], "data_split": "99,1,0"}
    with pytest.raises(ValueError):
        parse_cli_overrides(["novalue"])


def test_help_config_lists_fields(capsys):
    print_help_config()
    out = capsys.readouterr().out
    assert "learning_rate" in out and "Total:" in out and "MINTEXT_<FIELD_NAME_UPPER>" in out


def test_shipped_configs_load():
    from pathlib import Path

    root = Path(__file__).resolve().parents[1] / "configs"
    for f in sorted(root.glob("*/*.yml")):
        c = load_config(f)
        assert c.num_hidden_layers >= 1, f


def test_benchmark_configs_build_an_eight_gpu_mesh():
    """Every shipped benchmark config must give a valid mesh on the eight ranks it is written for."""
    from pathlib import Path

    from mintext_b200.parallel.mesh import create_mesh

    root = Path(__file__).resolve().parents[1] / "configs" / "benchmarks"
    files = sorted(root.glob("*.yml"))
    assert len(files) >= 4
    for f in files:
        c = load_config(f)
        m = create_mesh(c, devices=list(range(8)))
        assert m.size == 8, f
        assert (m.shape["data"] * m.shape["fsdp"]) % m.shape["expert"] == 0, f
        if c.num_experts > 0:
            assert m.shape["expert"] == 8 and c.num_experts % 8 == 0, f
            assert len(m.expert_group_ranks(3)) == 8
    c = load_config(root / "llama-3-8b-b200.yml")
    assert c.use_fp8 and str(c.fp8_recipe) == "mx_block" and c.ici_tensor_parallelism == 2


def test_bench_model_configs_split_the_batch():
    import importlib.util
    from pathlib import Path

    spec = importlib.util.spec_from_file_location("bench", Path(__file__).resolve().parents[1] / "bench.py")
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    for name, (yml, gb, _, _) in bench.BENCH_MODELS.items():
        cfg, got = bench.yaml_config(name, 8, None, None, None, 6, [])
        tp = cfg.ici_tensor_parallelism
        assert got == gb
        assert cfg.gradient_accumulation_steps * cfg.per_device_batch_size * (8 // tp) == gb, name
    cfg, _ = bench.yaml_config("qwen3moe", 2, 8, None, None, 6, ["num_experts=32", "ici_expert_parallelism=2"])
    assert cfg.num_experts == 32 and cfg.ici_expert_parallelism == 2


def test_layer_type_generation():
    assert MinTextConfig(model_type="qwen3_next", num_hidden_layers=8).layer_types.count("full_attention") == 2
    g = MinTextConfig(model_type="gemma3", num_hidden_layers=12).layer_types
    assert g[5] == "full_attention" and g[0] == "sliding_attention"
    q = MinTextConfig(model_type="qwen3", num_hidden_layers=4, use_sliding_window=True, max_window_layers=2).layer_types
    assert q == ["sliding_attention", "sliding_attention", "full_attention", "full_attention"]
