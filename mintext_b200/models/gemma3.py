"""Gemma 3: ``sliding_window_pattern - 1`` local layers followed by one global layer, repeated
(reference: mintext/models/gemma3.py:8-18)."""


def layer_types(num_hidden_layers: int, data: dict) -> list[str]:
    every = data.get("sliding_window_pattern", 6)
    return ["full_attention" if (i + 1) % every == 0 else "sliding_attention" for i in range(num_hidden_layers)]


get_layer_types = layer_types  # the reference's name for the per-family function
