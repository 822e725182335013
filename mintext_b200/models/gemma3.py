"""Gemma 3: ``sliding_window_pattern - 1`` local layers followed by one global layer, repeated
(reference: mintext/models/gemma3.py:8-18)."""


def layer_types(num_layers: int, cfg: dict) -> list[str]:
    every = cfg.get("sliding_window_pattern", 6)
    return ["full_attention" if (i + 1) % every == 0 else "sliding_attention" for i in range(num_layers)]
