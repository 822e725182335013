"""Qwen3-Next hybrid stack: every ``full_attention_interval``-th layer is gated full attention, the rest are
Gated-Delta-Rule linear attention (reference: mintext/models/qwen3_next.py:8-14)."""


def layer_types(num_layers: int, cfg: dict) -> list[str]:
    every = cfg.get("full_attention_interval", 4)
    return ["full_attention" if (i + 1) % every == 0 else "linear_attention" for i in range(num_layers)]
