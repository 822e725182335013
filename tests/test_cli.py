"""The training loop end to end through the public entry points (CPU plumbing path): config files + overrides,
synthetic batches, metric logging, checkpoints on the save interval, resume."""

import json
from pathlib import Path

import pytest

from mintext_b200.config import load_config
from mintext_b200.train import main, train

ROOT = Path(__file__).resolve().parents[1]
TINY = [str(ROOT / "configs" / "base.yml"), str(ROOT / "configs" / "models" / "test-tiny.yml")]


def _cfg(tmp_path, **kw):
    over = dict(steps=4, seq_length=32, per_device_batch_size=2, enable_tensorboard=False, log_period=1,
                checkpoint_dir=str(tmp_path / "ckpt"), enable_checkpointing=True, checkpoint_period=2,
                dtype="float32", weight_dtype="float32", kernel_backend="oracle", learning_rate=1e-3)
    over.update(kw)
    return load_config(TINY, over)


def test_train_loop_checkpoints_and_resumes(tmp_path):
    last = train(_cfg(tmp_path))
    assert last["step"] == 3 and last["loss"] == last["loss"]
    saved = sorted(int(p.name) for p in (tmp_path / "ckpt").iterdir() if p.name.isdigit())
    assert 4 in saved and 2 in saved, saved
    # a longer run from the same directory starts at the saved step and ends at its own last step
    last2 = train(_cfg(tmp_path, steps=6))
    assert last2["step"] == 5
    saved = sorted(int(p.name) for p in (tmp_path / "ckpt").iterdir() if p.name.isdigit())
    assert 6 in saved


def test_resumed_run_equals_uninterrupted_run(tmp_path):
    import shutil

    full = train(_cfg(tmp_path, steps=6, checkpoint_period=3))
    shutil.rmtree(tmp_path / "ckpt" / "6")  # as if the run had stopped after the step-3 checkpoint
    resumed = train(_cfg(tmp_path, steps=6, checkpoint_period=3))
    assert abs(full["loss"] - resumed["loss"]) < 1e-5, (full, resumed)


def test_cli_main_with_overrides(tmp_path, capsys):
    main(["--config", TINY[0], "--config", TINY[1], "steps=2", "seq_length=16", "enable_tensorboard=false",
          "enable_checkpointing=false", "kernel_backend=oracle", "dtype=float32", "weight_dtype=float32",
          f"log_dir={tmp_path}"])
    main(["--help-config"])
    assert "learning_rate" in capsys.readouterr().out


@pytest.mark.parametrize("model", ["deepseek-v3-4l", "qwen3-next-80b-a3b", "gemma-3-4b"])
def test_model_configs_shrink_and_train(tmp_path, model):
    """The shipped model configs, shrunk by overrides, run through the loop (MoE bias update included)."""
    paths = [str(ROOT / "configs" / "base.yml"), str(ROOT / "configs" / "models" / f"{model}.yml")]
    over = dict(steps=2, seq_length=16, per_device_batch_size=1, num_hidden_layers=2, hidden_size=64, vocab_size=128,
                num_attention_heads=4, num_key_value_heads=2, head_dim=16, intermediate_size=128,
                enable_tensorboard=False, enable_checkpointing=False, dtype="float32", weight_dtype="float32",
                kernel_backend="oracle", ici_expert_parallelism=1, ici_tensor_parallelism=1, ici_fsdp_parallelism=1,
                ici_data_parallelism=1)
    cfg0 = load_config(paths, None)
    if cfg0.num_experts > 0:
        over.update(num_experts=4, num_experts_per_tok=2, moe_intermediate_size=32, n_group=1, topk_group=1,
                    first_k_dense_replace=min(1, cfg0.first_k_dense_replace))
    if cfg0.attention_type == "mla":
        over.update(q_lora_rank=16, kv_lora_rank=16, qk_nope_head_dim=8, qk_rope_head_dim=4, v_head_dim=8)
    if model.startswith("qwen3-next"):
        over.update(linear_key_head_dim=8, linear_value_head_dim=8, linear_num_key_heads=2, linear_num_value_heads=4)
    if model.startswith("gemma"):
        over.update(sliding_window=8)
    last = train(load_config(paths, over))
    assert last["loss"] == last["loss"]


def test_cpu_plumbing_config_runs_ten_steps_and_learns():
    """The shipped CPU plumbing config (tiny Llama-style decoder, fp32, batch 8 x 128, AdamW, 10 steps)."""
    cfg = load_config(ROOT / "configs" / "benchmarks" / "test-tiny-cpu.yml")
    assert (cfg.num_hidden_layers, cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads) == (2, 128, 4, 2)
    assert (cfg.vocab_size, cfg.per_device_batch_size, cfg.seq_length, cfg.steps) == (1024, 8, 128, 10)
    last = train(cfg)
    assert last["step"] == 9 and last["loss"] == last["loss"] and last["loss"] < 7.5


def test_reference_module_paths_and_names_resolve():
    """Import paths and helper names of the reference package layout that differ from this package's own layout."""
    import importlib

    import torch

    mesh = importlib.import_module("mintext.distributed.mesh")
    assert mesh is importlib.import_module("mintext_b200.parallel.mesh") and hasattr(mesh, "create_mesh")
    assert hasattr(importlib.import_module("mintext.distributed.sharding"), "logical_to_pspec")
    assert hasattr(importlib.import_module("mintext.distributed.partition"), "create_sharded_model")
    base = importlib.import_module("mintext.models.base")
    from mintext_b200.models.transformer import Transformer

    assert base.Transformer is Transformer and callable(base._apply_layer_with_remat)
    for fam in ("llama3", "qwen3", "deepseek_v3", "qwen3_next", "gemma3"):
        mod = importlib.import_module(f"mintext.models.{fam}")
        assert len(mod.get_layer_types(4, {})) == 4
    from mintext.modules.linear import variance_scaling_init

    w = variance_scaling_init(2.0)(torch.Generator().manual_seed(0), (64, 4, 8), torch.float32, 0, (1, 2))
    assert w.shape == (64, 4, 8) and float(w.abs().max()) <= 2.0 * 2.0 / 8.0 + 1e-6   # |z| <= 2, fan_in = 64
    assert 0.15 < float(w.std()) < 0.25                                              # ~ 0.88 * 2 / 8


def test_reference_keyword_argument_names_are_accepted():
    """Calls written against the reference with keyword arguments keep working."""
    import inspect

    import torch

    from mintext import MinTextConfig
    from mintext.data.tokenizer import Tokenizer
    from mintext.distributed.sharding import create_named_sharding, get_model_param_shardings, logical_to_pspec
    from mintext.kernels import grouped_matmul, unroute
    from mintext.kernels.autotuner import autotune_moe
    from mintext.modules.attention import make_sliding_window_mask
    from mintext.modules.rope import RotaryEmbedding
    from mintext.trainer import chunked_cross_entropy_loss
    from mintext.utils.filesize import parse_file_size
    from mintext.utils.pytree import check_nan

    expected = {
        logical_to_pspec: ["logical_names", "rules", "mesh"],
        create_named_sharding: ["mesh", "logical_names", "rules"],
        get_model_param_shardings: ["model", "mesh", "rules"],
        grouped_matmul: ["x", "weights", "group_sizes", "tiling"],
        unroute: ["sorted_output", "sort_indices", "topk_weights", "num_experts_per_tok"],
        autotune_moe: ["config", "cache_dir", "max_trials", "warmup_iters", "bench_iters"],
        make_sliding_window_mask: ["seq_len", "window_size", "dtype"],
        chunked_cross_entropy_loss: ["hidden_states", "targets", "output_proj", "num_tiles", "label_smoothing",
                                     "z_loss_weight"],
        parse_file_size: ["size_str"],
        check_nan: ["tree", "label"],
        Tokenizer.__init__: ["self", "path", "type"],
        RotaryEmbedding.forward: ["self", "inputs", "positions"],
    }
    for fn, names in expected.items():
        have = list(inspect.signature(fn).parameters)
        assert have[:len(names)] == names, (fn.__qualname__, have)
    assert parse_file_size(size_str="2K") == 2048
    assert not check_nan(tree={"a": torch.ones(2)}, label="x") and check_nan(tree=[torch.tensor(float("nan"))])
    assert make_sliding_window_mask(seq_len=4, window_size=2).shape[-2:] == (4, 4)
    c = MinTextConfig(dtype="float32")
    assert c.jnp_dtype is torch.float32 and c.jnp_weight_dtype is torch.float32


def test_param_shardings_take_the_reference_argument_order():
    from mintext_b200 import MinTextConfig
    from mintext_b200.models import Transformer
    from mintext_b200.parallel import create_mesh, get_logical_axis_rules, get_model_param_shardings

    c = MinTextConfig(dtype="float32", vocab_size=64, num_hidden_layers=1, hidden_size=32, num_attention_heads=4,
                      num_key_value_heads=2, intermediate_size=64, seq_length=16)
    model = Transformer(c, rngs=0)
    mesh = create_mesh(MinTextConfig(ici_fsdp_parallelism=2, ici_tensor_parallelism=2), devices=list(range(4)))
    a = get_model_param_shardings(model, mesh)                                  # default rules
    b = get_model_param_shardings(model, mesh, get_logical_axis_rules(c))       # (model, mesh, rules)
    d = get_model_param_shardings(model, c, mesh)                               # (model, config, mesh)
    assert {k: v.spec for k, v in a.items()} == {k: v.spec for k, v in b.items()} == {k: v.spec for k, v in d.items()}
    assert a["layers.0.mlp.gate.kernel"].spec == ("fsdp", "tensor")
