"""Model families and the per-family layer-type registry.

``get_layer_types`` is importable without torch so that the config module can call it while validating.
"""

from __future__ import annotations

from typing import Any

from . import deepseek_v3, gemma3, llama3, qwen3, qwen3_next

_REGISTRY = {
    "llama3": llama3.layer_types,
    "qwen3": qwen3.layer_types,
    "deepseek_v3": deepseek_v3.layer_types,
    "qwen3_next": qwen3_next.layer_types,
    "gemma3": gemma3.layer_types,
}


def get_layer_types(model_type: str, num_hidden_layers: int, data: dict[str, Any]) -> list[str]:
    try:
        fn = _REGISTRY[str(model_type)]
    except KeyError:
        raise ValueError(f"Unknown model_type: {model_type}") from None
    return fn(num_hidden_layers, data)


def __getattr__(name: str):
    if name in ("Transformer", "DecoderLayer", "make_causal_mask", "_all_layers_scannable"):
        from . import transformer

        return getattr(transformer, name)
    raise AttributeError(name)


__all__ = ["get_layer_types", "Transformer", "DecoderLayer", "make_causal_mask", "_all_layers_scannable"]
