"""Llama 2/3: every layer is full causal attention (reference: mintext/models/llama3.py)."""


def layer_types(num_hidden_layers: int, data: dict) -> list[str]:
    return ["full_attention"] * num_hidden_layers


get_layer_types = layer_types  # the reference's name for the per-family function
