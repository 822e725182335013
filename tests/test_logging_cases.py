"""Single-behaviour tests of the utilities around the loop: parameter counting, the NaN check, the FLOP accounting,
the metric logger and the profiler window (after the cases of the reference's tests/test_logging.py)."""

import json
from pathlib import Path

import pytest
import torch

from mintext_b200 import MinTextConfig
from mintext_b200.utils import (MetricLogger, Profiler, calculate_tflops_per_device, calculate_tokens_per_device,
                                check_nan, count_params)


# ---- count_params / check_nan ------------------------------------------------------------------------------------
def test_count_params_flat():
    assert count_params({"a": torch.zeros(3, 4), "b": torch.zeros(5)}) == 17


def test_count_params_nested():
    assert count_params({"a": {"b": {"c": torch.zeros(2, 2)}}, "d": [torch.zeros(3)]}) == 7


def test_count_params_empty():
    assert count_params({}) == 0


def test_check_nan_clean_tree():
    assert not check_nan({"a": torch.ones(3), "b": {"c": torch.zeros(2)}})


def test_check_nan_finds_a_nan():
    assert check_nan({"a": torch.tensor([1.0, float("nan")])})


def test_check_nan_finds_a_nested_nan():
    assert check_nan({"a": torch.ones(2), "b": {"c": {"d": torch.tensor([float("nan")])}}})


def test_check_nan_ignores_integer_tensors():
    assert not check_nan({"ids": torch.arange(4)})


# ---- FLOP accounting ---------------------------------------------------------------------------------------------
def test_flops_of_a_small_llama_are_positive():
    assert calculate_tflops_per_device(MinTextConfig()) > 0


def test_a_larger_model_costs_more():
    small = calculate_tflops_per_device(MinTextConfig(hidden_size=128, num_hidden_layers=2))
    big = calculate_tflops_per_device(MinTextConfig(hidden_size=256, num_hidden_layers=4))
    assert big > 2 * small


def test_flops_scale_with_the_sequence_length_faster_than_linearly():
    a = calculate_tflops_per_device(MinTextConfig(seq_length=128))
    b = calculate_tflops_per_device(MinTextConfig(seq_length=256))
    assert b > 2 * a  # the attention term is quadratic


def test_moe_flops_count_the_active_experts_only():
    dense = MinTextConfig(intermediate_size=512)
    moe2 = MinTextConfig(num_experts=8, num_experts_per_tok=2, moe_intermediate_size=256, first_k_dense_replace=0)
    moe4 = moe2.model_copy(update={"num_experts_per_tok": 4})
    more_experts = moe2.model_copy(update={"num_experts": 16})
    assert calculate_tflops_per_device(moe4) > calculate_tflops_per_device(moe2)
    # twice the experts at the same top-k only adds the wider router
    assert calculate_tflops_per_device(more_experts) < 1.05 * calculate_tflops_per_device(moe2)
    assert calculate_tflops_per_device(dense) > 0


def test_mla_flops_are_positive():
    c = MinTextConfig(attention_type="mla", q_lora_rank=32, kv_lora_rank=16, qk_nope_head_dim=16, qk_rope_head_dim=8,
                      v_head_dim=16)
    assert calculate_tflops_per_device(c) > 0


def test_gradient_accumulation_scales_the_flops():
    one = calculate_tflops_per_device(MinTextConfig())
    four = calculate_tflops_per_device(MinTextConfig(gradient_accumulation_steps=4))
    assert four == pytest.approx(4 * one)


def test_tokens_per_device():
    assert calculate_tokens_per_device(MinTextConfig(per_device_batch_size=4, seq_length=64)) == 256


def test_tokens_per_device_with_accumulation():
    c = MinTextConfig(per_device_batch_size=4, seq_length=64, gradient_accumulation_steps=3)
    assert calculate_tokens_per_device(c) == 768


# ---- metric logger -----------------------------------------------------------------------------------------------
def _step(lg, step=0):
    lg.log_step(step, {"loss": 2.0, "learning_rate": 1e-3, "grad_norm": 0.7, "param_norm": 3.0}, 0.5)


def test_logger_without_tensorboard(tmp_path):
    lg = MetricLogger(MinTextConfig(enable_tensorboard=False, base_output_directory=str(tmp_path)))
    _step(lg)
    lg.close()
    assert not Path(lg.config.tensorboard_dir).exists() if hasattr(lg, "config") else True


def test_logger_with_tensorboard_writes_event_files(tmp_path):
    pytest.importorskip("tensorboard")
    c = MinTextConfig(enable_tensorboard=True, base_output_directory=str(tmp_path))
    lg = MetricLogger(c)
    _step(lg)
    lg.close()
    assert any(Path(c.tensorboard_dir).iterdir())


def test_logger_writes_one_json_line_per_step(tmp_path):
    c = MinTextConfig(enable_tensorboard=False, base_output_directory=str(tmp_path))
    lg = MetricLogger(c)
    for s in range(3):
        _step(lg, s)
    lg.close()
    lines = (Path(c.log_dir) / "metrics.jsonl").read_text().splitlines()
    assert [json.loads(l)["step"] for l in lines] == [0, 1, 2]


def test_logger_json_record_fields(tmp_path):
    c = MinTextConfig(enable_tensorboard=False, base_output_directory=str(tmp_path))
    lg = MetricLogger(c)
    _step(lg, 5)
    lg.close()
    rec = json.loads((Path(c.log_dir) / "metrics.jsonl").read_text().splitlines()[-1])
    assert rec["loss"] == 2.0 and rec["grad_norm"] == 0.7 and rec["step_time"] == 0.5
    assert rec["tokens_per_sec_per_device"] == pytest.approx(calculate_tokens_per_device(c) / 0.5)
    assert rec["tflops_per_device"] == pytest.approx(calculate_tflops_per_device(c) / 0.5)


def test_logger_console_line(tmp_path, caplog):
    lg = MetricLogger(MinTextConfig(enable_tensorboard=False, base_output_directory=str(tmp_path)))
    with caplog.at_level("INFO", logger="mintext_b200"):
        _step(lg, 7)
    lg.close()
    assert "step=7" in caplog.text and "loss=2.0000" in caplog.text and "TFLOP/s/device=" in caplog.text


def test_logger_reports_the_parameter_count(tmp_path, caplog):
    with caplog.at_level("INFO", logger="mintext_b200"):
        lg = MetricLogger(MinTextConfig(enable_tensorboard=False, base_output_directory=str(tmp_path)),
                          params={"w": torch.zeros(1000, 1000)})
    lg.close()
    assert "1,000,000" in caplog.text or "1000000" in caplog.text or "1.00" in caplog.text


def test_logger_tolerates_a_zero_step_time(tmp_path):
    lg = MetricLogger(MinTextConfig(enable_tensorboard=False, base_output_directory=str(tmp_path)))
    lg.log_step(0, {"loss": 1.0, "learning_rate": 0.0, "grad_norm": 0.0}, 0.0)
    lg.close()


# ---- profiler window ---------------------------------------------------------------------------------------------
def test_profiler_disabled_never_activates():
    p = Profiler(MinTextConfig(enable_profiler=False))
    for s in range(5):
        p.maybe_activate(s)
        assert not p.active


def test_profiler_window_bounds(tmp_path):
    c = MinTextConfig(enable_profiler=True, skip_first_n_profiler_steps=2, profiler_steps=3, base_output_directory=str(tmp_path))
    p = Profiler(c)
    assert (p.start_step, p.end_step) == (2, 5) and p.output_dir.endswith("profiles")


def test_profiler_activates_at_its_first_step_only(tmp_path):
    c = MinTextConfig(enable_profiler=True, skip_first_n_profiler_steps=2, profiler_steps=2, base_output_directory=str(tmp_path))
    p = Profiler(c)
    p.maybe_activate(0)
    p.maybe_activate(1)
    assert not p.active
    p.maybe_activate(2)
    assert p.active
    p.maybe_deactivate(2)
    assert p.active
    p.maybe_deactivate(3)
    assert not p.active
    assert (Path(p.output_dir) / "trace.json").exists()


def test_profiler_stop_is_idempotent(tmp_path):
    c = MinTextConfig(enable_profiler=True, skip_first_n_profiler_steps=0, profiler_steps=1, base_output_directory=str(tmp_path))
    p = Profiler(c)
    p.maybe_activate(0)
    p.stop()
    p.stop()
    assert not p.active
