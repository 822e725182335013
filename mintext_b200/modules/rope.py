"""Rotary embeddings: default, linear, YaRN and Llama-3 frequency scaling; half-rotation or interleaved pairing;
partial rotary (reference: mintext/modules/rope.py)."""

from __future__ import annotations

import torch
from torch import nn

from mintext_b200.ops import functional as F
from mintext_b200.ops.oracle import compute_inv_freq as _compute_inv_freq
from mintext_b200.ops.oracle import rope_tables


def compute_inv_freq(config, dim: int):
    """``(inv_freq[dim/2], attention_factor)`` for the config's ``rope_type``."""
    return _compute_inv_freq(config, dim)


class RotaryEmbedding(nn.Module):
    """Input ``[B, S, H, head_dim]``, positions ``[B, S]``."""

    def __init__(self, config, rope_dim: int | None = None, theta: float | None = None):
        super().__init__()
        head_dim = rope_dim if rope_dim is not None else config.head_dim
        self.head_dim = head_dim
        self.interleave = bool(config.rope_interleave)
        rot = head_dim
        if config.partial_rotary_factor < 1.0:
            rot = int(head_dim * config.partial_rotary_factor)
            rot -= rot % 2
        self._rot_dim = rot
        inv, att = _compute_inv_freq(config, rot, theta)
        self.register_buffer("_inv_freq", inv, persistent=False)
        self._attention_factor = float(att)
        self._max_pos = int(config.seq_length)
        self._tables = None

    def _cuda_tables(self, device, need: int):
        if self._tables is None or self._tables[0].device != device or self._tables[0].shape[0] < need:
            n = max(need, self._max_pos)
            self._tables = rope_tables(self._inv_freq.float().cpu(), self._attention_factor, n, device=device)
        return self._tables

    def forward(self, inputs: torch.Tensor, positions: torch.Tensor | None,
                default_positions: bool = False) -> torch.Tensor:
        x = inputs
        tables = self._cuda_tables(x.device, x.shape[1]) if F.use_cuda(x) else None
        return F.rope(x, positions, self._inv_freq, self._attention_factor, self._rot_dim, self.interleave,
                      tables=tables, default_positions=default_positions)
