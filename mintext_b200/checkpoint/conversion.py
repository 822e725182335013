"""HuggingFace safetensors import / export (reference: mintext/checkpoint/conversion.py).

The correspondence between HF tensor names and this framework's parameter tree is a table of
``(hf name, our name, transform)`` rows produced from the config (one block of rows per layer, chosen by the
layer's attention and feed-forward kind).  A transform is a short code with an exact inverse:

    id          same tensor
    T           2-D transpose                      HF Linear [out, in]          <-> kernel [in, out]
    qkv:h,d     head-expanding projection          HF [(h*d), D]                <-> kernel [D, h, d]
    out:h,d     head-contracting projection        HF [D, (h*d)]                <-> kernel [h, d, D]
    norm1       RMSNorm stored as (w - 1) in HF    HF w                          <-> scale = w + 1

Routed experts are handled apart from the table: HF stores ``mlp.experts.{e}.{gate,up,down}_proj.weight`` (or the
fused ``mlp.experts.gate_up_proj [E, 2I, D]`` / ``mlp.experts.down_proj [E, D, I]``); here they live in
``mlp.experts.gate_up_proj [E, D, 2I]`` (gate columns first) and ``mlp.experts.down_proj [E, I, D]``.
"""

from __future__ import annotations

import json
import logging
from pathlib import Path
from typing import Callable

import torch

logger = logging.getLogger(__name__)

Row = tuple[str, str, str]


# ------------------------------------------------------------------------------------------- transforms
def _apply(code: str, t: torch.Tensor, inverse: bool = False) -> torch.Tensor:
    if code == "id":
        return t
    if code == "T":
        return t.t().contiguous()
    if code == "norm1":
        return t - 1.0 if inverse else t + 1.0
    kind, args = code.split(":")
    h, d = (int(x) for x in args.split(","))
    if kind == "qkv":
        if inverse:  # [D, h, d] -> [(h d), D]
            return t.permute(1, 2, 0).reshape(h * d, -1).contiguous()
        return t.reshape(h, d, -1).permute(2, 0, 1).contiguous()
    if kind == "out":
        if inverse:  # [h, d, D] -> [D, (h d)]
            return t.reshape(h * d, -1).t().contiguous()
        return t.t().reshape(h, d, -1).contiguous()
    raise ValueError(f"unknown transform {code}")


# kept under the reference's helper names for tests that exercise single transforms
def _transpose(t: torch.Tensor) -> torch.Tensor:
    return _apply("T", t)


def _rmsnorm_hf_to_mt(t: torch.Tensor) -> torch.Tensor:
    return _apply("norm1", t)


def _rmsnorm_mt_to_hf(t: torch.Tensor) -> torch.Tensor:
    return _apply("norm1", t, inverse=True)


# ------------------------------------------------------------------------------------------- key table
def _layer_rows(config, i: int) -> list[Row]:
    hf, mt = f"model.layers.{i}", f"layers.{i}"
    mtype = config.model_type
    H, Hkv, dh = config.num_attention_heads, config.num_key_value_heads or config.num_attention_heads, config.head_dim
    layer_type = config.layer_types[i] if i < len(config.layer_types) else "full_attention"
    norm = "norm1" if mtype in ("qwen3_next", "gemma3") else "id"
    rows: list[Row] = []

    # attention
    if layer_type == "linear_attention":
        la = f"{hf}.linear_attn"
        rows += [(f"{la}.in_proj_qkvz.weight", f"{mt}.attention.in_proj_qkvz.kernel", "T"),
                 (f"{la}.in_proj_ba.weight", f"{mt}.attention.in_proj_ba.kernel", "T"),
                 (f"{la}.conv1d.weight", f"{mt}.attention.conv_weight", "id"),
                 (f"{la}.A_log", f"{mt}.attention.A_log", "id"),
                 (f"{la}.dt_bias", f"{mt}.attention.dt_bias", "id"),
                 (f"{la}.norm.weight", f"{mt}.attention.norm.scale", "id"),  # gated norm: plain weight
                 (f"{la}.out_proj.weight", f"{mt}.attention.out_proj.kernel", "T")]
    elif config.attention_type == "mla":
        sa = f"{hf}.self_attn"
        qk, vd, nope = config.qk_head_dim, config.v_head_dim, config.qk_nope_head_dim
        if config.q_lora_rank > 0:
            rows += [(f"{sa}.q_a_proj.weight", f"{mt}.attention.q_a_proj.kernel", "T"),
                     (f"{sa}.q_a_layernorm.weight", f"{mt}.attention.q_a_norm.scale", "id"),
                     (f"{sa}.q_b_proj.weight", f"{mt}.attention.q_b_proj.kernel", f"qkv:{H},{qk}")]
        else:
            rows += [(f"{sa}.q_proj.weight", f"{mt}.attention.q_proj.kernel", f"qkv:{H},{qk}")]
        rows += [(f"{sa}.kv_a_proj_with_mqa.weight", f"{mt}.attention.kv_a_proj.kernel", "T"),
                 (f"{sa}.kv_a_layernorm.weight", f"{mt}.attention.kv_a_norm.scale", "id"),
                 (f"{sa}.kv_b_proj.weight", f"{mt}.attention.kv_b_proj.kernel", f"qkv:{H},{nope + vd}"),
                 (f"{sa}.o_proj.weight", f"{mt}.attention.out.kernel", f"out:{H},{vd}")]
    else:
        sa = f"{hf}.self_attn"
        gated = mtype == "qwen3_next"
        rows += [(f"{sa}.q_proj.weight", f"{mt}.attention.query.kernel", f"qkv:{H},{2 * dh if gated else dh}"),
                 (f"{sa}.k_proj.weight", f"{mt}.attention.key.kernel", f"qkv:{Hkv},{dh}"),
                 (f"{sa}.v_proj.weight", f"{mt}.attention.value.kernel", f"qkv:{Hkv},{dh}"),
                 (f"{sa}.o_proj.weight", f"{mt}.attention.out.kernel", f"out:{H},{dh}")]
        if config.use_qk_norm:
            qk_norm = "norm1" if mtype in ("qwen3_next", "gemma3") else "id"
            rows += [(f"{sa}.q_norm.weight", f"{mt}.attention.q_norm.scale", qk_norm),
                     (f"{sa}.k_norm.weight", f"{mt}.attention.k_norm.scale", qk_norm)]

    # feed-forward
    if config.num_experts > 0 and i >= config.first_k_dense_replace:
        rows.append((f"{hf}.mlp.gate.weight", f"{mt}.mlp.router.gate.kernel", "T"))
        if config.router_type == "sigmoid_group":
            rows.append((f"{hf}.mlp.gate.e_score_correction_bias", f"{mt}.mlp.router.e_score_correction_bias", "id"))
        if config.n_shared_experts > 0:
            # HF Qwen3-Next names its (gated) shared expert in the singular; DeepSeek-V3 uses the plural
            shared = "shared_expert" if config.shared_expert_gate else "shared_experts"
            for a, b in (("gate_proj", "gate"), ("up_proj", "up"), ("down_proj", "down")):
                rows.append((f"{hf}.mlp.{shared}.{a}.weight", f"{mt}.mlp.shared_expert.{b}.kernel", "T"))
            if config.shared_expert_gate:
                rows.append((f"{hf}.mlp.shared_expert_gate.weight", f"{mt}.mlp.shared_expert_gate.kernel", "T"))
    else:
        for a, b in (("gate_proj", "gate"), ("up_proj", "up"), ("down_proj", "down")):
            rows.append((f"{hf}.mlp.{a}.weight", f"{mt}.mlp.{b}.kernel", "T"))

    # norms
    rows += [(f"{hf}.input_layernorm.weight", f"{mt}.pre_attn_norm.scale", norm),
             (f"{hf}.post_attention_layernorm.weight", f"{mt}.post_attn_norm.scale", norm)]
    if config.use_post_ffw_norm:
        rows += [(f"{hf}.pre_feedforward_layernorm.weight", f"{mt}.pre_ffw_norm.scale", norm),
                 (f"{hf}.post_feedforward_layernorm.weight", f"{mt}.post_ffw_norm.scale", norm)]
    return rows


def key_table(config) -> list[Row]:
    norm = "norm1" if config.model_type in ("qwen3_next", "gemma3") else "id"
    rows: list[Row] = [("model.embed_tokens.weight", "token_embedder", "id")]
    for i in range(config.num_hidden_layers):
        rows += _layer_rows(config, i)
    rows += [("model.norm.weight", "final_norm.scale", norm), ("lm_head.weight", "output_proj.kernel", "T")]
    return rows


def _hf_to_mintext_key_map(config) -> dict[str, tuple[str, Callable | None]]:
    """``{hf key: (our key, transform or None)}``."""
    return {hf: (mt, None if code == "id" else (lambda t, c=code: _apply(c, t))) for hf, mt, code in key_table(config)}


def _mintext_to_hf_key_map(config) -> dict[str, tuple[str, Callable | None]]:
    """``{our key: (hf key, inverse transform or None)}``."""
    return {mt: (hf, None if code == "id" else (lambda t, c=code: _apply(c, t, inverse=True)))
            for hf, mt, code in key_table(config)}


# ------------------------------------------------------------------------------------------- tree helpers
def _flatten_state(model: torch.nn.Module) -> dict[str, torch.Tensor]:
    """``{dotted name: tensor}`` of every parameter."""
    return {n: p.detach() for n, p in model.named_parameters()}


def _moe_layers(config) -> list[int]:
    if config.num_experts <= 0:
        return []
    return [i for i in range(config.num_hidden_layers) if i >= config.first_k_dense_replace]


def _import_experts(hf: dict[str, torch.Tensor], config, dtype) -> dict[str, torch.Tensor]:
    out: dict[str, torch.Tensor] = {}
    E = config.num_experts
    for i in _moe_layers(config):
        base = f"model.layers.{i}.mlp.experts"
        fused_gu, fused_dn = hf.get(f"{base}.gate_up_proj"), hf.get(f"{base}.down_proj")
        if fused_gu is not None and fused_dn is not None:
            out[f"layers.{i}.mlp.experts.gate_up_proj"] = fused_gu.transpose(1, 2).contiguous().to(dtype)
            out[f"layers.{i}.mlp.experts.down_proj"] = fused_dn.transpose(1, 2).contiguous().to(dtype)
            continue
        if f"{base}.0.gate_proj.weight" not in hf:
            continue
        gu = [torch.cat([hf[f"{base}.{e}.gate_proj.weight"].t(), hf[f"{base}.{e}.up_proj.weight"].t()], dim=1)
              for e in range(E)]
        dn = [hf[f"{base}.{e}.down_proj.weight"].t() for e in range(E)]
        out[f"layers.{i}.mlp.experts.gate_up_proj"] = torch.stack(gu).contiguous().to(dtype)
        out[f"layers.{i}.mlp.experts.down_proj"] = torch.stack(dn).contiguous().to(dtype)
    return out


def _export_experts(state: dict[str, torch.Tensor], config) -> dict[str, torch.Tensor]:
    out: dict[str, torch.Tensor] = {}
    I = config.moe_intermediate_size
    for i in _moe_layers(config):
        gu = state.get(f"layers.{i}.mlp.experts.gate_up_proj")
        dn = state.get(f"layers.{i}.mlp.experts.down_proj")
        if gu is None or dn is None:
            continue
        base = f"model.layers.{i}.mlp.experts"
        for e in range(gu.shape[0]):
            out[f"{base}.{e}.gate_proj.weight"] = gu[e, :, :I].t().contiguous()
            out[f"{base}.{e}.up_proj.weight"] = gu[e, :, I:].t().contiguous()
            out[f"{base}.{e}.down_proj.weight"] = dn[e].t().contiguous()
    return out


# ------------------------------------------------------------------------------------------- import / export
@torch.no_grad()
def load_hf_checkpoint(hf_path: str, config, model: torch.nn.Module) -> torch.nn.Module:
    """Fill ``model``'s parameters from every ``*.safetensors`` file in ``hf_path``.  Shapes are checked;
    missing and unused keys are logged."""
    from safetensors.torch import load_file

    files = sorted(Path(hf_path).glob("*.safetensors"))
    if not files:
        raise FileNotFoundError(f"No .safetensors files found in {hf_path}")
    hf: dict[str, torch.Tensor] = {}
    for f in files:
        hf.update(load_file(str(f)))
    params = dict(model.named_parameters())
    loaded, used = set(), set()
    for hf_key, mt_key, code in key_table(config):
        if hf_key not in hf:
            continue
        used.add(hf_key)
        if mt_key not in params:
            continue
        t = _apply(code, hf[hf_key].float())
        p = params[mt_key]
        if tuple(t.shape) != tuple(p.shape):
            raise ValueError(f"Shape mismatch for {mt_key}: checkpoint {tuple(t.shape)} vs model {tuple(p.shape)}")
        p.copy_(t.to(p.dtype))
        loaded.add(mt_key)
    for mt_key, t in _import_experts(hf, config, torch.float32).items():
        if mt_key in params:
            if tuple(t.shape) != tuple(params[mt_key].shape):
                raise ValueError(f"Shape mismatch for {mt_key}: {tuple(t.shape)} vs {tuple(params[mt_key].shape)}")
            params[mt_key].copy_(t.to(params[mt_key].dtype))
            loaded.add(mt_key)
    used |= {k for k in hf if ".mlp.experts." in k}
    missing = sorted(set(params) - loaded)
    if config.tie_word_embeddings:
        missing = [m for m in missing if m != "output_proj.kernel"]
    extra = sorted(set(hf) - used)
    if missing:
        logger.warning("Parameters not found in the HF checkpoint (left at init): %s", missing[:20])
    if extra:
        logger.info("HF tensors without a counterpart (ignored): %s", extra[:20])
    return model


def save_hf_checkpoint(model: torch.nn.Module, config, output_path: str, hf_config: dict | None = None) -> None:
    """Write ``model.safetensors`` + ``config.json`` that ``transformers`` loads with ``from_pretrained``."""
    from safetensors.torch import save_file

    out_dir = Path(output_path)
    out_dir.mkdir(parents=True, exist_ok=True)
    state = {n: t.float().cpu() for n, t in _flatten_state(model).items()}
    tensors: dict[str, torch.Tensor] = {}
    for hf_key, mt_key, code in key_table(config):
        if mt_key in state:
            tensors[hf_key] = _apply(code, state[mt_key], inverse=True).contiguous()
    tensors.update(_export_experts(state, config))
    if config.tie_word_embeddings:
        tensors.pop("lm_head.weight", None)
    save_file(tensors, str(out_dir / "model.safetensors"), metadata={"format": "pt"})
    with open(out_dir / "config.json", "w") as f:
        json.dump(hf_config or _mintext_to_hf_config(config), f, indent=2)


# ------------------------------------------------------------------------------------------- HF config.json
def _rope_scaling(config) -> dict | None:
    rt = config.rope_type
    if rt == "default":
        return None
    if rt == "linear":
        return {"rope_type": "linear", "factor": config.rope_scaling_factor}
    if rt == "llama3":
        return {"rope_type": "llama3", "factor": config.rope_scaling_factor,
                "low_freq_factor": config.rope_llama3_low_freq_factor,
                "high_freq_factor": config.rope_llama3_high_freq_factor,
                "original_max_position_embeddings": config.rope_original_max_position_embeddings or config.seq_length}
    return {"rope_type": "yarn", "factor": config.rope_scaling_factor, "beta_fast": config.rope_yarn_beta_fast,
            "beta_slow": config.rope_yarn_beta_slow, "mscale": config.rope_yarn_mscale,
            "mscale_all_dim": config.rope_yarn_mscale_all_dim,
            "original_max_position_embeddings": config.rope_original_max_position_embeddings or config.seq_length}


def _mintext_to_hf_config(config) -> dict:
    """A ``config.json`` dict for the matching ``transformers`` architecture."""
    c = config
    common = {
        "hidden_size": c.hidden_size, "num_hidden_layers": c.num_hidden_layers,
        "num_attention_heads": c.num_attention_heads, "num_key_value_heads": c.num_key_value_heads,
        "intermediate_size": c.intermediate_size, "vocab_size": c.vocab_size, "rms_norm_eps": c.rms_norm_eps,
        "max_position_embeddings": c.seq_length, "tie_word_embeddings": c.tie_word_embeddings,
        "rope_theta": c.rope_theta, "hidden_act": c.hidden_activation, "torch_dtype": "float32",
        "attention_bias": False,
    }
    rs = _rope_scaling(c)
    if rs is not None:
        common["rope_scaling"] = rs
    mt = c.model_type
    if mt == "llama3":
        return {**common, "architectures": ["LlamaForCausalLM"], "model_type": "llama", "head_dim": c.head_dim,
                "mlp_bias": False}
    if mt == "qwen3":
        return {**common, "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "head_dim": c.head_dim,
                "use_sliding_window": c.use_sliding_window, "sliding_window": c.sliding_window,
                "max_window_layers": c.max_window_layers, "layer_types": list(c.layer_types)}
    if mt == "deepseek_v3":
        return {**common, "num_key_value_heads": c.num_attention_heads,
                "architectures": ["DeepseekV3ForCausalLM"], "model_type": "deepseek_v3",
                "q_lora_rank": c.q_lora_rank if c.q_lora_rank > 0 else None, "kv_lora_rank": c.kv_lora_rank,
                "qk_nope_head_dim": c.qk_nope_head_dim, "qk_rope_head_dim": c.qk_rope_head_dim,
                "v_head_dim": c.v_head_dim, "n_routed_experts": c.num_experts,
                "num_experts_per_tok": c.num_experts_per_tok, "moe_intermediate_size": c.moe_intermediate_size,
                "n_shared_experts": c.n_shared_experts, "n_group": c.n_group, "topk_group": c.topk_group,
                "first_k_dense_replace": c.first_k_dense_replace, "routed_scaling_factor": c.routed_scaling_factor,
                "norm_topk_prob": c.norm_topk_prob, "rope_interleave": c.rope_interleave, "moe_layer_freq": 1}
    if mt == "qwen3_next":
        return {**common, "architectures": ["Qwen3NextForCausalLM"], "model_type": "qwen3_next",
                "head_dim": c.head_dim, "partial_rotary_factor": c.partial_rotary_factor,
                "full_attention_interval": c.full_attention_interval, "layer_types": list(c.layer_types),
                "linear_key_head_dim": c.linear_key_head_dim, "linear_value_head_dim": c.linear_value_head_dim,
                "linear_num_key_heads": c.linear_num_key_heads, "linear_num_value_heads": c.linear_num_value_heads,
                "linear_conv_kernel_dim": c.linear_conv_kernel_dim, "num_experts": c.num_experts,
                "num_experts_per_tok": c.num_experts_per_tok, "moe_intermediate_size": c.moe_intermediate_size,
                "shared_expert_intermediate_size": c.moe_intermediate_size * max(c.n_shared_experts, 1),
                "norm_topk_prob": c.norm_topk_prob, "decoder_sparse_step": 1, "mlp_only_layers":
                list(range(c.first_k_dense_replace))}
    if mt == "gemma3":
        return {**common, "architectures": ["Gemma3ForCausalLM"], "model_type": "gemma3_text", "head_dim": c.head_dim,
                "hidden_activation": c.hidden_activation, "query_pre_attn_scalar": int(c.query_pre_attn_scalar or c.head_dim),
                "attn_logit_softcapping": c.attn_logit_softcapping,
                "final_logit_softcapping": c.final_logit_softcapping, "sliding_window": c.sliding_window,
                "sliding_window_pattern": c.sliding_window_pattern, "rope_local_base_freq": c.rope_local_theta,
                "layer_types": list(c.layer_types)}
    raise ValueError(f"Unknown model_type: {mt}")
