"""Qwen3-Next hybrid stack: every ``full_attention_interval``-th layer is gated full attention, the rest are
Gated-Delta-Rule linear attention (reference: mintext/models/qwen3_next.py:8-14)."""


def layer_types(num_hidden_layers: int, data: dict) -> list[str]:
    every = data.get("full_attention_interval", 4)
    return ["full_attention" if (i + 1) % every == 0 else "linear_attention" for i in range(num_hidden_layers)]


get_layer_types = layer_types  # the reference's name for the per-family function
