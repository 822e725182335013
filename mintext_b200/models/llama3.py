"""Llama 2/3: every layer is full causal attention (reference: mintext/models/llama3.py)."""


def layer_types(num_layers: int, cfg: dict) -> list[str]:
    return ["full_attention"] * num_layers
