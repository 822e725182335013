"""DeepSeek-V3: full attention everywhere; MLA and MoE are switched by config fields, not by layer type
(reference: mintext/models/deepseek_v3.py)."""


def layer_types(num_hidden_layers: int, data: dict) -> list[str]:
    return ["full_attention"] * num_hidden_layers


get_layer_types = layer_types  # the reference's name for the per-family function
