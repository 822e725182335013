"""Configuration: one flat, frozen pydantic model plus the YAML / CLI / environment loader.

Parity target: ``mintext/config.py`` of the reference (field names, defaults, derived fields, validation
messages, override priority CLI > ``MINTEXT_<KEY>`` environment > YAML with recursive ``base_config``).
Differences: the YAML layer is PyYAML (no OmegaConf), several config files can be merged left to right,
``torch_dtype`` / ``torch_weight_dtype`` (also under the reference's names ``jnp_dtype`` / ``jnp_weight_dtype``) return
torch dtypes, and there are extra keys for the
parallel modes the reference does not have (expert parallelism, router type, fp8 recipe ...).
"""

from __future__ import annotations

import difflib
import enum
import logging
import os
from pathlib import Path
from typing import Any, Iterable

import yaml
from pydantic import BaseModel, ConfigDict, field_validator, model_validator

logger = logging.getLogger(__name__)

ENV_PREFIX = "MINTEXT_"


class _StrEnum(str, enum.Enum):
    def __str__(self) -> str:  # pragma: no cover - cosmetic
        return self.value


DType = _StrEnum("DType", {n: n for n in ("bfloat16", "float32", "float16")})
OptimizerType = _StrEnum("OptimizerType", {n: n for n in ("adamw", "muon")})
LRScheduleType = _StrEnum("LRScheduleType", {n: n for n in ("cosine", "linear", "wsd")})
RematPolicy = _StrEnum(
    "RematPolicy",
    {n: n for n in ("full", "minimal", "none", "save_qkv_proj", "save_dot_except_mlp", "qkv_proj_offloaded",
                    "minimal_offloaded")},
)
DatasetType = _StrEnum("DatasetType", {n: n for n in ("synthetic", "mmap", "arecord", "auto")})
ModelType = _StrEnum("ModelType", {n: n for n in ("llama3", "qwen3", "deepseek_v3", "qwen3_next", "gemma3")})
RopeType = _StrEnum("RopeType", {n: n for n in ("default", "llama3", "yarn", "linear")})
RouterType = _StrEnum("RouterType", {n: n for n in ("sigmoid_group", "softmax_topk")})
Fp8Recipe = _StrEnum("Fp8Recipe", {n: n for n in ("per_tensor", "mx_block")})

# logical axis -> mesh axis; the first matching rule wins.  ("exp" -> "expert" is this framework's addition:
# the reference keeps experts unsharded.)
DEFAULT_LOGICAL_AXIS_RULES: list[tuple[str, str | None]] = [
    ("batch", "data"),
    ("length", None),
    ("embed", "fsdp"),
    ("heads", "tensor"),
    ("q_heads", "tensor"),
    ("kv_heads", None),
    ("kv_head_dim", None),
    ("kv", None),
    ("mlp", "tensor"),
    ("vocab", "tensor"),
    ("norm", None),
    ("exp", None),
]

_POSITIVE = ("num_hidden_layers", "hidden_size", "num_attention_heads", "vocab_size", "per_device_batch_size")


class MinTextConfig(BaseModel):
    """All knobs of a run.  ``MinTextConfig()`` is a valid test-sized model."""

    model_config = ConfigDict(frozen=True, use_enum_values=True)

    # run
    run_name: str = "default"
    model_name: str = "test-tiny"
    base_output_directory: str = "/tmp/mintext"
    seed: int = 0

    # architecture
    num_hidden_layers: int = 2
    hidden_size: int = 128
    num_attention_heads: int = 4
    num_key_value_heads: int | None = None
    intermediate_size: int = 512
    head_dim: int | None = None
    vocab_size: int = 256
    rms_norm_eps: float = 1e-5
    seq_length: int = 128
    tie_word_embeddings: bool = False
    hidden_activation: str = "silu"
    model_type: ModelType = ModelType.llama3

    # qwen3
    use_qk_norm: bool = False
    use_sliding_window: bool = False
    sliding_window: int = 4096
    max_window_layers: int = 28
    layer_types: list[str] = []

    # multi-head latent attention (DeepSeek-V3)
    attention_type: str = "mha"
    q_lora_rank: int = 0
    kv_lora_rank: int = 512
    qk_nope_head_dim: int = 128
    qk_rope_head_dim: int = 64
    v_head_dim: int = 128
    rope_interleave: bool = False
    attention_causal_mla: bool = True  # False reproduces the reference's unmasked MLA training

    # mixture of experts
    num_experts: int = 0
    num_experts_per_tok: int = 8
    moe_intermediate_size: int = 2048
    n_shared_experts: int = 1
    n_group: int = 8
    topk_group: int = 4
    first_k_dense_replace: int = 3
    routed_scaling_factor: float = 2.5
    norm_topk_prob: bool = True
    e_score_correction_bias_update_rate: float = 0.001
    router_type: RouterType = RouterType.sigmoid_group
    router_aux_loss_coef: float = 0.0
    shared_expert_gate: bool = False  # Qwen3-Next: shared expert output times sigmoid(x @ w_gate)
    moe_use_custom_vjp: bool = True
    moe_mosaic_fusion_group: bool = True
    moe_autotune: bool = False
    moe_autotune_cache_dir: str = ""
    moe_gate_up_tiling: list[int] = []
    moe_down_tiling: list[int] = []
    moe_use_fp8: bool = False
    moe_capacity_factor: float = 2.0  # expert-parallel receive buffers hold this multiple of a rank's own rows

    # qwen3-next
    full_attention_interval: int = 4
    partial_rotary_factor: float = 1.0
    linear_key_head_dim: int = 128
    linear_value_head_dim: int = 128
    linear_num_key_heads: int | None = None
    linear_num_value_heads: int | None = None
    linear_conv_kernel_dim: int = 4

    # gemma3
    query_pre_attn_scalar: float | None = None
    attn_logit_softcapping: float | None = None
    final_logit_softcapping: float | None = None
    sliding_window_pattern: int = 6
    rope_local_theta: float = 10_000.0
    use_post_ffw_norm: bool = False
    scale_embeddings: bool = False

    # dtypes
    dtype: DType = DType.bfloat16
    weight_dtype: DType = DType.float32

    # rotary embeddings
    rope_type: RopeType = RopeType.default
    rope_theta: float = 10_000.0
    rope_scaling_factor: float = 1.0
    rope_original_max_position_embeddings: int = 0
    rope_yarn_beta_fast: float = 32.0
    rope_yarn_beta_slow: float = 1.0
    rope_yarn_mscale: float = 1.0
    rope_yarn_mscale_all_dim: float = 0.0
    rope_llama3_low_freq_factor: float = 1.0
    rope_llama3_high_freq_factor: float = 4.0

    # loop
    num_vocab_tiles: int = 1
    steps: int = 10
    log_period: int = 1
    label_smoothing: float = 0.0
    eval_period: int = 0  # > 0: run eval_step on the eval split every N steps (the reference never evaluates)
    eval_steps: int = 1
    synthetic_shift_targets: bool = False  # False: targets == inputs, as the reference's synthetic batches

    # optimizer
    shard_optimizer_over_data: bool = False
    optimizer: OptimizerType = OptimizerType.adamw
    learning_rate: float = 1e-3
    lr_schedule: LRScheduleType = LRScheduleType.cosine
    warmup_steps_fraction: float = 0.1
    lr_final_fraction: float = 0.1
    gradient_accumulation_steps: int = 1
    gradient_clip_threshold: float = 1.0
    adam_b1: float = 0.9
    adam_b2: float = 0.95
    adam_eps: float = 1e-8
    weight_decay: float = 0.1
    wsd_decay_steps_fraction: float = 0.1
    wsd_decay_style: str = "linear"
    z_loss_weight: float = 0.0
    muon_newton_schulz_steps: int = 5
    muon_beta: float = 0.95
    muon_consistent_rms: float | None = None

    # memory / kernels
    remat_policy: RematPolicy = RematPolicy.none
    use_custom_kernels: bool = False
    use_fp8: bool = False
    fp8_recipe: Fp8Recipe = Fp8Recipe.per_tensor
    kernel_backend: str = "auto"  # auto | cuda | oracle
    # draw the initial weights on the GPU (seeded from `seed`); "auto": when the model has more than 2e9 parameters,
    # where host-side sampling by every rank would take minutes and tens of GB of host memory per process
    init_weights_on_device: str = "auto"  # auto | true | false
    # synthetic batches: "threefry" = counter-based stream keyed by `seed`, split once per step, every rank writing
    # its own rows of the global batch on the device; "torch" = the host generator (one stream per data-parallel rank)
    synthetic_rng: str = "threefry"

    # data
    dataset_type: DatasetType = DatasetType.synthetic
    per_device_batch_size: int = 2
    data_path: str = ""
    data_cache_dir: str = ""
    data_split: str = "99,1,0"
    num_data_epochs: int = 1
    add_extra_token: bool = True
    grain_worker_count: int = 4
    grain_prefetch_buffer_size: int = 500

    # mesh
    ici_data_parallelism: int = 1
    ici_fsdp_parallelism: int = -1
    ici_tensor_parallelism: int = 1
    ici_expert_parallelism: int = 1
    scan_layers: bool = True
    dcn_data_parallelism: int = 1
    dcn_fsdp_parallelism: int = 1
    dcn_tensor_parallelism: int = 1
    num_slices: int = 1
    jax_distributed_init_timeout: int = 300
    # failure detection (none of this exists in the reference): peer heartbeats over the job's store, checked before
    # every step (0 = off), and what to do with a NaN / Inf loss: ignore | skip | abort
    heartbeat_interval: float = 0.0
    heartbeat_timeout: float = 60.0
    nan_policy: str = "ignore"
    logical_axis_rules: list[tuple[str, str | None]] = []
    fused_collectives: bool = True  # peer-memory kernels for the sharded optimizer step; False: NCCL composition
    # layer weights and layer gradients sharded 1/N over data x fsdp (gathered one layer ahead, reduce-scattered per
    # layer) instead of resident on every rank: parallel/fsdp.py.  "auto": sharded when the resident copies (2 + 4 bytes
    # per parameter a rank holds) would exceed `fsdp_resident_budget_gb` per GPU.
    fsdp_shard_params: bool | str = False
    fsdp_resident_budget_gb: float = 60.0
    # under tensor parallelism: shard the embedding table and the output head over the vocabulary as well (the
    # reference's `vocab -> tensor` rule): parallel/vocab_parallel.py.  Off: both are whole on every rank of the group
    # and work on the rank's token shard through the fused projection + loss kernel.
    tp_vocab_parallel: bool = False

    # checkpoints
    enable_checkpointing: bool = True
    async_checkpointing: bool = True
    checkpoint_period: int = 1000
    checkpoint_dir: str = ""
    max_checkpoints: int = 5
    load_checkpoint: str = ""
    load_hf_checkpoint: str = ""
    load_params_only: bool = False

    # accepted for compatibility with reference configs; no effect on a GPU
    tpu_type: str = "auto"
    xla_flags: str = ""

    # logging / profiling
    enable_tensorboard: bool = True
    tensorboard_dir: str = ""
    log_dir: str = ""
    enable_profiler: bool = False
    profiler_steps: int = 5
    skip_first_n_profiler_steps: int = 1

    # ------------------------------------------------------------------ derived values
    @property
    def qk_head_dim(self) -> int:
        return self.qk_nope_head_dim + self.qk_rope_head_dim

    @property
    def torch_dtype(self):
        import torch

        return getattr(torch, self.dtype)

    @property
    def torch_weight_dtype(self):
        import torch

        return getattr(torch, self.weight_dtype)

    # the reference's property names (mintext/config.py: jnp_dtype / jnp_weight_dtype); the values are torch dtypes
    jnp_dtype = torch_dtype
    jnp_weight_dtype = torch_weight_dtype

    # ------------------------------------------------------------------ validation
    @field_validator("rope_type", mode="before")
    @classmethod
    def _rope_alias(cls, v: Any) -> Any:
        return "llama3" if v == "llama3_1" else v

    @field_validator("fsdp_shard_params", mode="before")
    @classmethod
    def _normalise_shard_mode(cls, v):
        if isinstance(v, str):
            low = v.strip().lower()
            if low in ("true", "1", "yes"):
                return True
            if low in ("false", "0", "no", ""):
                return False
            if low == "auto":
                return "auto"
            raise ValueError(f"fsdp_shard_params must be true, false or auto, got '{v}'")
        return v

    @field_validator(*_POSITIVE)
    @classmethod
    def _at_least_one(cls, v: int, info) -> int:
        if v < 1:
            raise ValueError(f"{info.field_name} must be >= 1, got {v}")
        return v

    @field_validator("steps")
    @classmethod
    def _steps_ok(cls, v: int) -> int:
        if v < 0:
            raise ValueError(f"steps must be >= 0, got {v}")
        return v

    @model_validator(mode="before")
    @classmethod
    def _fill_derived(cls, data: Any) -> Any:
        if not isinstance(data, dict):
            return data
        data = dict(data)
        heads = data.get("num_attention_heads", 4)
        if data.get("head_dim") is None and heads and heads > 0:
            data["head_dim"] = data.get("hidden_size", 128) // heads
        for key in ("num_key_value_heads", "linear_num_key_heads", "linear_num_value_heads"):
            if data.get(key) is None:
                data[key] = heads
        if not data.get("layer_types"):
            from mintext_b200.models import get_layer_types

            data["layer_types"] = get_layer_types(
                str(getattr(data.get("model_type", "llama3"), "value", data.get("model_type", "llama3"))),
                data.get("num_hidden_layers", 2),
                data,
            )
        if not data.get("logical_axis_rules"):
            data["logical_axis_rules"] = list(DEFAULT_LOGICAL_AXIS_RULES)
        root = os.path.join(data.get("base_output_directory", "/tmp/mintext"), data.get("run_name", "default"))
        for key, leaf in (("checkpoint_dir", "checkpoints"), ("tensorboard_dir", "tensorboard"), ("log_dir", "logs")):
            if not data.get(key):
                data[key] = os.path.join(root, leaf)
        return data

    @model_validator(mode="after")
    def _cross_field_checks(self) -> "MinTextConfig":
        if self.num_vocab_tiles > 1:
            tokens = self.per_device_batch_size * self.seq_length
            if tokens % self.num_vocab_tiles != 0:
                raise ValueError(
                    f"per_device_batch_size * seq_length ({tokens}) must be "
                    f"divisible by num_vocab_tiles ({self.num_vocab_tiles})"
                )
        if self.load_checkpoint and self.load_hf_checkpoint:
            raise ValueError("`load_checkpoint` and `load_hf_checkpoint` are mutually exclusive.")
        if self.load_params_only and not self.load_checkpoint:
            raise ValueError("`load_params_only` requires `load_checkpoint` to be set.")
        return self


# ---------------------------------------------------------------------------- loading
def _read_yaml_with_bases(path: Path, _seen: tuple[Path, ...] = ()) -> dict[str, Any]:
    """One YAML file merged over the chain of files its ``base_config`` keys point to."""
    path = path.resolve()
    if path in _seen:
        raise ValueError(f"base_config cycle through {path}")
    with open(path) as f:
        data = yaml.safe_load(f) or {}
    if not isinstance(data, dict):
        raise ValueError(f"Config file {path} must be a YAML mapping")
    parent = data.pop("base_config", None)
    if parent is None:
        return data
    parent_path = Path(parent)
    if not parent_path.is_absolute():
        parent_path = path.parent / parent_path
    merged = _read_yaml_with_bases(parent_path, _seen + (path,))
    merged.update(data)
    return merged


def _reject_unknown(keys: Iterable[str]) -> None:
    known = set(MinTextConfig.model_fields)
    unknown = sorted(set(keys) - known)
    if not unknown:
        return
    lines = []
    for key in unknown:
        close = difflib.get_close_matches(key, known, n=1, cutoff=0.6)
        lines.append(f"  '{key}' (did you mean '{close[0]}'?)" if close else f"  '{key}'")
    raise ValueError("Unknown config key(s):\n" + "\n".join(lines))


def _coerce_env(key: str, raw: str, current: Any, present: bool) -> Any:
    if key == "fsdp_shard_params" and raw.strip().lower() == "auto":
        return "auto"
    if isinstance(current, bool) or (current is None and present):
        low = raw.lower()
        if low in ("true", "1", "yes"):
            return True
        if low in ("false", "0", "no"):
            return False
        raise ValueError(f"Cannot parse '{raw}' as bool for env var '{ENV_PREFIX + key.upper()}'")
    if isinstance(current, int):
        return int(raw)
    if isinstance(current, float):
        return float(raw)
    return raw


def _merge_environment(data: dict[str, Any], cli_keys: frozenset[str]) -> dict[str, Any]:
    for key in MinTextConfig.model_fields:
        raw = os.environ.get(ENV_PREFIX + key.upper())
        if raw is None:
            continue
        if key in cli_keys:
            raise ValueError(
                f"Key '{key}' is overridden by both CLI and environment variable "
                f"'{ENV_PREFIX + key.upper()}'. Remove one to avoid ambiguity."
            )
        data[key] = _coerce_env(key, raw, data.get(key), key in data)
        logger.info("Config '%s' overridden by env var %s=%s", key, ENV_PREFIX + key.upper(), raw)
    return data


def parse_cli_overrides(items: Iterable[str]) -> dict[str, Any]:
    """``key=value`` tokens -> dict; values are typed the way YAML scalars / flow sequences are."""
    out: dict[str, Any] = {}
    for item in items:
        if "=" not in item:
            raise ValueError(f"Expected key=value, got '{item}'")
        key, raw = item.split("=", 1)
        key = key.strip().lstrip("-")
        try:
            value = yaml.safe_load(raw) if raw != "" else ""
        except yaml.YAMLError:
            value = raw
        # YAML reads 1e-4 as a string; accept the common float spellings
        if isinstance(value, str):
            try:
                value = float(value) if any(c in value for c in "eE.") and value.strip() else value
            except ValueError:
                pass
        out[key] = value
    return out


def load_config(config_path: str | Path | list[str | Path], overrides: dict[str, Any] | None = None) -> MinTextConfig:
    """Build a validated config.  Priority: ``overrides`` (CLI) > ``MINTEXT_*`` environment > YAML chain.

    ``config_path`` may be a list; the files are merged left to right (each one still follows its own
    ``base_config`` chain first).
    """
    paths = config_path if isinstance(config_path, (list, tuple)) else [config_path]
    data: dict[str, Any] = {}
    for p in paths:
        data.update(_read_yaml_with_bases(Path(p)))
    cli_keys: frozenset[str] = frozenset()
    if overrides:
        _reject_unknown(overrides)
        cli_keys = frozenset(overrides)
        data.update(overrides)
    data = _merge_environment(data, cli_keys)
    return MinTextConfig(**data)


def print_help_config() -> None:
    """Table of every field with its type and default."""
    fields = MinTextConfig.model_fields
    print("MinText Configuration Fields")
    print("=" * 72)
    print(f"{'Field':<35} {'Type':<20} {'Default'}")
    print("-" * 72)
    for name, info in fields.items():
        ann = info.annotation
        tname = getattr(ann, "__name__", str(ann)).replace("typing.", "")
        if len(tname) > 18:
            tname = tname[:17] + "…"
        default = info.default
        if isinstance(default, str) and len(default) > 30:
            default = default[:27] + "..."
        print(f"  {name:<33} {tname:<20} {default}")
    print()
    print(f"Total: {len(fields)} fields")
    print()
    print("Environment variable override: MINTEXT_<FIELD_NAME_UPPER>=value")
    print("  Example: MINTEXT_LEARNING_RATE=1e-4")
