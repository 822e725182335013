"""Utilities: parameter counting, NaN check, FLOP accounting, metric logger, profiler window, file sizes."""

import pytest
import torch

from mintext_b200 import MinTextConfig
from mintext_b200.utils import (MetricLogger, Profiler, calculate_tflops_per_device, calculate_tokens_per_device,
                                check_nan, count_params, parse_file_size)


def test_count_params_and_nan():
    tree = {"a": torch.zeros(3, 4), "b": {"c": torch.zeros(5)}}
    assert count_params(tree) == 17
    assert not check_nan(tree)
    tree["b"]["c"][2] = float("nan")
    assert check_nan(tree)


def test_flops_formula_scaling():
    base = MinTextConfig()
    f0 = calculate_tflops_per_device(base)
    assert f0 > 0
    assert calculate_tflops_per_device(MinTextConfig(num_hidden_layers=4)) > f0
    assert calculate_tflops_per_device(MinTextConfig(gradient_accumulation_steps=2)) == pytest.approx(2 * f0)
    moe = MinTextConfig(num_experts=8, num_experts_per_tok=2, moe_intermediate_size=256, first_k_dense_replace=1)
    assert calculate_tflops_per_device(moe) > 0
    mla = MinTextConfig(attention_type="mla", q_lora_rank=32, kv_lora_rank=16, qk_nope_head_dim=16,
                        qk_rope_head_dim=8, v_head_dim=16)
    assert calculate_tflops_per_device(mla) > 0
    assert calculate_tokens_per_device(MinTextConfig(per_device_batch_size=4, seq_length=64)) == 256


def test_flops_llama_1b_matches_published_accounting():
    c = MinTextConfig(num_hidden_layers=16, hidden_size=2048, num_attention_heads=32, num_key_value_heads=8,
                      head_dim=64, intermediate_size=8192, vocab_size=128256, seq_length=4096,
                      per_device_batch_size=64)
    per_token = calculate_tflops_per_device(c) * 1e12 / (64 * 4096) / 1e9
    assert per_token == pytest.approx(8.22, abs=0.02)  # GFLOP per token


def test_metric_logger_console_and_jsonl(tmp_path, caplog):
    c = MinTextConfig(enable_tensorboard=False, base_output_directory=str(tmp_path))
    lg = MetricLogger(c, params={"w": torch.zeros(10)})
    with caplog.at_level("INFO", logger="mintext_b200"):
        lg.log_step(3, {"loss": 1.5, "learning_rate": 1e-3, "grad_norm": 0.5, "param_norm": 2.0}, 0.25)
    lg.close()
    text = caplog.text
    assert "step=3" in text and "loss=1.5000" in text and "MFU=" in text and "tokens/s/device=" in text
    import json
    from pathlib import Path

    rec = json.loads((Path(c.log_dir) / "metrics.jsonl").read_text().splitlines()[-1])
    assert rec["step"] == 3 and rec["loss"] == 1.5


def test_metric_logger_tensorboard(tmp_path):
    pytest.importorskip("tensorboard")
    c = MinTextConfig(enable_tensorboard=True, base_output_directory=str(tmp_path))
    lg = MetricLogger(c)
    lg.log_step(0, {"loss": 1.0, "learning_rate": 1e-3, "grad_norm": 1.0}, 0.1)
    lg.close()
    from pathlib import Path

    assert any(Path(c.tensorboard_dir).iterdir())


def test_profiler_window(tmp_path):
    c = MinTextConfig(enable_profiler=True, profiler_steps=2, skip_first_n_profiler_steps=1,
                      base_output_directory=str(tmp_path))
    p = Profiler(c)
    p.maybe_activate(0)
    assert not p.active
    p.maybe_activate(1)
    assert p.active
    p.maybe_deactivate(1)
    assert p.active
    p.maybe_deactivate(2)
    assert not p.active
    off = Profiler(MinTextConfig())
    off.maybe_activate(1)
    assert not off.active


@pytest.mark.parametrize("text,expected", [("5G", 5 * 1024 ** 3), ("100MB", 100 * 1024 ** 2), ("1.5g", int(1.5 * 1024 ** 3)),
                                           ("2k", 2048), (1048576, 1048576), ("123", 123)])
def test_parse_file_size(text, expected):
    assert parse_file_size(text) == expected


def test_parse_file_size_errors():
    for bad in ("abc", "5X", ""):
        with pytest.raises(ValueError):
            parse_file_size(bad)


def test_per_device_throughput_counts_a_tensor_parallel_group_once():
    """``per_device_batch_size`` sequences belong to one data-parallel rank, i.e. to a whole tensor-parallel group."""
    base = dict(per_device_batch_size=2, seq_length=64, gradient_accumulation_steps=3)
    one = MinTextConfig(**base)
    two = MinTextConfig(**base, ici_tensor_parallelism=2, ici_fsdp_parallelism=1)
    assert calculate_tokens_per_device(one) == 2 * 64 * 3
    assert calculate_tokens_per_device(two) == 2 * 64 * 3 / 2
    assert abs(calculate_tflops_per_device(two) - calculate_tflops_per_device(one) / 2) < 1e-12
