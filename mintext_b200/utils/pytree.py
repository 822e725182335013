"""Parameter counting, NaN checks and the analytic FLOP / token accounting used for TFLOP/s and MFU
(reference: mintext/utils/pytree.py).

The FLOP count deliberately matches the reference's MaxText-style formula term by term (it ignores linear-
attention layers, sliding windows and shared experts, and prices MLA scores with ``head_dim``), because MFU is
only comparable when both sides use the same numerator.
"""

from __future__ import annotations

from typing import Iterable

import torch


def _leaves(params) -> Iterable[torch.Tensor]:
    if isinstance(params, torch.nn.Module):
        return list(params.parameters())
    if isinstance(params, dict):
        out = []
        for v in params.values():
            out.extend(_leaves(v) if isinstance(v, (dict, list, tuple)) else [v])
        return out
    if isinstance(params, (list, tuple)):
        return list(params)
    return [params]


def count_params(params) -> int:
    return sum(int(t.numel()) for t in _leaves(params) if isinstance(t, torch.Tensor))


def check_nan(tree, label: str = "params") -> bool:
    """True when any leaf holds a NaN or an infinity (``label`` is accepted for signature parity and unused, as in
    mintext/utils/pytree.py:16-25)."""
    params = tree
    return any(not bool(torch.isfinite(t.float()).all()) for t in _leaves(params) if isinstance(t, torch.Tensor))


def model_flops_per_token_batch(config, batch: int) -> float:
    """Forward+backward FLOPs of one step over ``batch`` sequences of ``seq_length`` tokens."""
    B, S, D, V, L = batch, config.seq_length, config.hidden_size, config.vocab_size, config.num_hidden_layers
    H = config.num_attention_heads
    Hkv = config.num_key_value_heads or H
    dh = config.head_dim or D // H
    dense_ffn = 2 * B * S * D * config.intermediate_size * 3
    if config.num_experts > 0:
        moe_layers = max(0, L - config.first_k_dense_replace)
        router = 2 * B * S * D * config.num_experts
        expert = 2 * B * S * D * config.moe_intermediate_size * 3
        ffn = dense_ffn * (L - moe_layers) + (router + expert * config.num_experts_per_tok) * moe_layers
    else:
        ffn = dense_ffn * L
    if config.attention_type == "mla":
        proj = 2 * B * S * (
            D * config.q_lora_rank + config.q_lora_rank * H * config.qk_head_dim
            + D * (config.kv_lora_rank + config.qk_rope_head_dim)
            + config.kv_lora_rank * H * (config.qk_nope_head_dim + config.v_head_dim)
            + H * config.v_head_dim * D)
    else:
        proj = 2 * B * S * D * ((H + 2 * Hkv) * dh + H * dh)
    scores = 4 * B * S * S * H * dh // 2
    head = 2 * B * S * D * V
    return float((ffn + (proj + scores) * L + head) * 3)


def estimate_param_count(config) -> float:
    """Approximate number of parameters of the model a config describes (embedding, projections, feed-forward
    weights; norms and biases ignored).  Used to pick host- or device-side initialisation before anything is built."""
    D, V, L = config.hidden_size, config.vocab_size, config.num_hidden_layers
    H = config.num_attention_heads
    Hkv = config.num_key_value_heads or H
    dh = config.head_dim or D // H
    if config.attention_type == "mla":
        attn = (D * config.q_lora_rank + config.q_lora_rank * H * config.qk_head_dim
                + D * (config.kv_lora_rank + config.qk_rope_head_dim)
                + config.kv_lora_rank * H * (config.qk_nope_head_dim + config.v_head_dim) + H * config.v_head_dim * D)
    else:
        attn = D * (H + 2 * Hkv) * dh + H * dh * D
    dense = 3 * D * config.intermediate_size
    if config.num_experts > 0:
        moe_layers = max(0, L - config.first_k_dense_replace)
        moe = D * config.num_experts + 3 * D * config.moe_intermediate_size * (
            config.num_experts + config.n_shared_experts)
        ffn = dense * (L - moe_layers) + moe * moe_layers
    else:
        ffn = dense * L
    emb = V * D * (1 if config.tie_word_embeddings else 2)
    return float(emb + attn * L + ffn)


def resident_param_bytes_per_rank(config) -> float:
    """Bytes a rank holds in the resident engine mode for the bf16 compute copy and the fp32 gradient accumulator
    (6 per parameter): dense parameters in full (divided by the tensor-parallel degree where they are sliced: an
    upper bound, embeddings are not), routed experts divided by the expert-parallel degree."""
    total = estimate_param_count(config)
    experts = 0.0
    if config.num_experts > 0:
        moe_layers = max(0, config.num_hidden_layers - config.first_k_dense_replace)
        experts = 3.0 * config.hidden_size * config.moe_intermediate_size * config.num_experts * moe_layers
    ep = max(int(getattr(config, "ici_expert_parallelism", 1) or 1), 1)
    dense = (total - experts) / _tensor_parallel_degree(config)
    return 6.0 * (dense + experts / ep)


def wants_sharded_params(config, world: int) -> bool:
    """Decision behind ``fsdp_shard_params``: explicit true / false, or ``"auto"``: shard when there is more than one
    data-parallel rank to shard over, the configuration is one the sharded mode covers (AdamW, bf16, peer-memory
    collectives, no tensor parallelism) and the resident copies would take more than ``fsdp_resident_budget_gb``."""
    mode = config.fsdp_shard_params
    if isinstance(mode, str):
        low = mode.strip().lower()
        if low in ("true", "1", "yes"):
            return True
        if low in ("false", "0", "no", ""):
            return False
        if low != "auto":
            raise ValueError(f"fsdp_shard_params must be true, false or auto, got '{mode}'")
        covered = (world > 1 and str(config.optimizer) == "adamw" and bool(config.fused_collectives)
                   and str(config.dtype) == "bfloat16" and _tensor_parallel_degree(config) == 1)
        return covered and resident_param_bytes_per_rank(config) > float(config.fsdp_resident_budget_gb) * 2 ** 30
    return bool(mode)


def _tensor_parallel_degree(config) -> int:
    dcn = int(getattr(config, "dcn_tensor_parallelism", 1) or 1)
    return max(int(getattr(config, "ici_tensor_parallelism", 1) or 1), 1) * max(dcn, 1)


def calculate_tflops_per_device(config) -> float:
    """TFLOP per device per optimizer step.  ``per_device_batch_size`` sequences per micro-step are processed by one
    data-parallel rank, i.e. by a whole tensor-parallel group: a device's share is 1 / tensor-parallel degree of it
    (the reference replicates work under its sharding instead and counts it in full, mintext/utils/pytree.py:35-37)."""
    per_group = model_flops_per_token_batch(config, config.per_device_batch_size) * config.gradient_accumulation_steps
    return per_group / _tensor_parallel_degree(config) / 1e12


def calculate_tokens_per_device(config) -> float:
    per_group = config.per_device_batch_size * config.seq_length * config.gradient_accumulation_steps
    return per_group / _tensor_parallel_degree(config)
