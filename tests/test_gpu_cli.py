"""`python -m mintext_b200.train` on the GPU: single-GPU run with checkpoint + resume, and two-GPU runs through
torch.distributed.run with tensor parallelism and with expert parallelism (fused peer-memory kernels on)."""

import os
import re
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]
BASE = ["--config", str(ROOT / "configs" / "base.yml"), "--config", str(ROOT / "configs" / "models" / "test-tiny.yml")]
COMMON = ["seq_length=128", "per_device_batch_size=4", "enable_tensorboard=false", "log_period=1", "learning_rate=1e-3",
          "hidden_size=256", "num_attention_heads=4", "num_key_value_heads=2", "head_dim=64", "vocab_size=1024"]


def _run(cmd, timeout=600):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=str(ROOT))
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=timeout, cwd=str(ROOT))
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    return r.stdout + r.stderr


def _losses(out):
    return [float(m) for m in re.findall(r"loss[=:]\s*([0-9.]+)", out)]


def test_single_gpu_cli_checkpoint_and_resume(tmp_path):
    args = BASE + COMMON + ["steps=6", f"checkpoint_dir={tmp_path}/ckpt", "checkpoint_period=3", "enable_checkpointing=true"]
    out = _run([sys.executable, "-m", "mintext_b200.train"] + args)
    first = _losses(out)
    assert len(first) >= 6 and all(0.0 < l < 12.0 for l in first), first   # fresh random batches: no trend expected
    saved = sorted(int(p.name) for p in (tmp_path / "ckpt").iterdir() if p.name.isdigit())
    assert saved == [3, 6], saved
    out2 = _run([sys.executable, "-m", "mintext_b200.train"] + args[:-4] + ["steps=8"] + args[-3:])
    second = _losses(out2)
    assert len(second) == 2 and all(0.0 < l < 12.0 for l in second), (first, second)   # resumed at step 6


@pytest.mark.parametrize("extra", [["ici_tensor_parallelism=2"],
                                   ["ici_expert_parallelism=2", "num_experts=4", "num_experts_per_tok=2",
                                    "moe_intermediate_size=128", "n_group=1", "topk_group=1", "first_k_dense_replace=1",
                                    "model_type=deepseek_v3", "attention_type=mha"],
                                   # tensor parallelism around sub-layers that run replicated (MLA, experts)
                                   ["ici_tensor_parallelism=2", "num_experts=4", "num_experts_per_tok=2",
                                    "moe_intermediate_size=128", "n_group=1", "topk_group=1", "first_k_dense_replace=1",
                                    "model_type=deepseek_v3", "attention_type=mla", "q_lora_rank=64", "kv_lora_rank=64",
                                    "qk_nope_head_dim=128", "qk_rope_head_dim=64", "v_head_dim=128"]])
def test_two_gpu_cli_tensor_and_expert_parallel(tmp_path, extra):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29681", "-m", "mintext_b200.train"] + BASE + COMMON + \
          ["steps=5", "enable_checkpointing=false", "fused_collectives=true"] + extra
    out = _run(cmd)
    losses = _losses(out)
    assert len(losses) >= 5 and all(0.0 < l < 12.0 for l in losses), losses
