"""RMSNorm with an fp32 scale initialised to ones (reference: mintext/modules/norm.py)."""

from __future__ import annotations

import torch
from torch import nn

from mintext_b200.ops import functional as F


class RMSNorm(nn.Module):
    def __init__(self, dim: int, epsilon: float = 1e-5, dtype: torch.dtype = torch.float32, *, rngs=None):
        super().__init__()
        self.dim = dim
        self.epsilon = epsilon
        self.dtype = dtype
        self.scale = nn.Parameter(torch.ones(dim, dtype=torch.float32))
        self.scale.logical_axes = ("norm",)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return F.rms_norm(x, self.scale, self.epsilon, self.dtype)

    def forward_add(self, x: torch.Tensor, residual: torch.Tensor):
        """Fused ``h = x + residual`` then norm; returns ``(norm(h), h)``."""
        return F.add_rms_norm(x, residual, self.scale, self.epsilon)
