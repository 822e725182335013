"""Qwen3: the first ``max_window_layers`` layers use sliding-window attention when ``use_sliding_window`` is
set, all others full attention (reference: mintext/models/qwen3.py:8-17)."""


def layer_types(num_hidden_layers: int, data: dict) -> list[str]:
    if not data.get("use_sliding_window", False):
        return ["full_attention"] * num_hidden_layers
    cut = data.get("max_window_layers", 28)
    return ["sliding_attention" if i < cut else "full_attention" for i in range(num_hidden_layers)]


get_layer_types = layer_types  # the reference's name for the per-family function
