"""DeepSeek-V3: full attention everywhere; MLA and MoE are switched by config fields, not by layer type
(reference: mintext/models/deepseek_v3.py)."""


def layer_types(num_layers: int, cfg: dict) -> list[str]:
    return ["full_attention"] * num_layers
