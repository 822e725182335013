"""Multi-head latent attention (DeepSeek-V3; reference: mintext/modules/mla.py).

Queries optionally go through a low-rank bottleneck (``q_a_proj -> q_a_norm -> q_b_proj``); keys/values are
expanded from a shared latent (``kv_a_proj -> kv_a_norm -> kv_b_proj``) and one rotary key part shared by all
heads.  Scale is ``(nope + rope) ** -0.5``.  Unlike the reference, which applies a mask only when one is passed
(and therefore trains bidirectionally), attention here is causal unless ``attention_causal_mla`` is False.
"""

from __future__ import annotations

import torch
from torch import nn

from mintext_b200.ops import functional as F

from .linear import Linear
from .norm import RMSNorm
from .rope import RotaryEmbedding


class MLAttention(nn.Module):
    def __init__(self, config, layer_idx: int = 0, *, rngs=None):
        super().__init__()
        self.num_attention_heads = H = config.num_attention_heads
        self.q_lora_rank = config.q_lora_rank
        self.kv_lora_rank = config.kv_lora_rank
        self.qk_nope_head_dim = config.qk_nope_head_dim
        self.qk_rope_head_dim = config.qk_rope_head_dim
        self.v_head_dim = config.v_head_dim
        self.causal = bool(config.attention_causal_mla)
        self.dtype = dt = config.torch_dtype
        wdt = config.torch_weight_dtype
        D = config.hidden_size
        qk = config.qk_head_dim
        self.scale = qk ** -0.5
        if self.q_lora_rank > 0:
            self.q_a_proj = Linear(D, self.q_lora_rank, dt, wdt, ("embed", "mlp"), rngs=rngs)
            self.q_a_norm = RMSNorm(self.q_lora_rank, config.rms_norm_eps, dt)
            self.q_b_proj = Linear(self.q_lora_rank, (H, qk), dt, wdt, ("embed", "heads", "kv"), rngs=rngs,
                                   name="query_proj")
        else:
            self.q_proj = Linear(D, (H, qk), dt, wdt, ("embed", "heads", "kv"), rngs=rngs, name="query_proj")
        self.kv_a_proj = Linear(D, self.kv_lora_rank + self.qk_rope_head_dim, dt, wdt, ("embed", "mlp"), rngs=rngs,
                                name="key_proj")
        self.kv_a_norm = RMSNorm(self.kv_lora_rank, config.rms_norm_eps, dt)
        self.kv_b_proj = Linear(self.kv_lora_rank, (H, self.qk_nope_head_dim + self.v_head_dim), dt, wdt,
                                ("embed", "heads", "kv"), rngs=rngs, name="value_proj")
        self.out = Linear((H, self.v_head_dim), D, dt, wdt, ("heads", "kv", "embed"), rngs=rngs, name="out_proj")
        self.rope = RotaryEmbedding(config, rope_dim=self.qk_rope_head_dim)

    def forward(self, x: torch.Tensor, positions: torch.Tensor | None, mask: torch.Tensor | None = None,
                default_positions: bool = False) -> torch.Tensor:
        B, S, _ = x.shape
        H = self.num_attention_heads
        if self.q_lora_rank > 0:
            q = self.q_b_proj(self.q_a_norm(self.q_a_proj(x)))
        else:
            q = self.q_proj(x)
        q_nope, q_rope = q.split([self.qk_nope_head_dim, self.qk_rope_head_dim], dim=-1)
        kv_c = self.kv_a_proj(x)
        latent, k_rope_raw = kv_c.split([self.kv_lora_rank, self.qk_rope_head_dim], dim=-1)
        kv = self.kv_b_proj(self.kv_a_norm(latent.contiguous()))
        k_nope, v = kv.split([self.qk_nope_head_dim, self.v_head_dim], dim=-1)
        q_rope = self.rope(q_rope.contiguous(), positions, default_positions)
        k_rope = self.rope(k_rope_raw.reshape(B, S, 1, self.qk_rope_head_dim).contiguous(), positions,
                           default_positions)
        qf = torch.cat([q_nope, q_rope], dim=-1)
        kf = torch.cat([k_nope, k_rope.expand(B, S, H, self.qk_rope_head_dim)], dim=-1)
        if mask is not None:
            o = F.attention(qf, kf, v, self.scale, causal=False, mask=mask)
        else:
            o = F.attention(qf, kf, v, self.scale, causal=self.causal)
        return self.out(o)
