"""Building blocks (the reference's ``mintext.modules`` surface)."""

from .attention import Attention, make_sliding_window_mask
from .linear import ACT2FN, MLP, Linear
from .linear_attention import GatedDeltaRuleAttention, chunk_gated_delta_rule
from .mla import MLAttention
from .moe import MoEBlock, MoEExperts, MoERouter
from .norm import RMSNorm
from .rope import RotaryEmbedding, compute_inv_freq

__all__ = [
    "RMSNorm", "Linear", "MLP", "ACT2FN", "Attention", "MLAttention", "make_sliding_window_mask",
    "GatedDeltaRuleAttention", "chunk_gated_delta_rule", "MoERouter", "MoEExperts", "MoEBlock",
    "RotaryEmbedding", "compute_inv_freq",
]
