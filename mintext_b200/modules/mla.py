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
        # Tensor parallelism: the per-head expansions (q_b / q, kv_b) are column-parallel over heads and the output
        # projection row-parallel; the low-rank down-projections and their norms stay whole on every rank and see
        # the gathered tokens, so each rank's gradient for them is the contribution of its own heads - a partial
        # sum that the engine's cross-rank gradient sum completes.
        from mintext_b200.parallel.tp import current_tp

        self.tp = current_tp() if (current_tp() is not None and current_tp().size > 1) else None
        self.local_heads = H
        if self.tp is not None:
            lo, hi = self.tp.shard(H, "num_attention_heads")
            self.local_heads = hi - lo
            heads_out = [self.q_b_proj if self.q_lora_rank > 0 else self.q_proj, self.kv_b_proj]
            for lin, dim in [(m, 1) for m in heads_out] + [(self.out, 0)]:
                full = lin.kernel.data
                axes = lin.kernel.logical_axes
                lin.kernel = nn.Parameter((full[:, lo:hi] if dim == 1 else full[lo:hi]).clone().contiguous())
                lin.kernel.logical_axes = axes
                lin.kernel.tensor_parallel = True
                lin.kernel.shard_spec = (dim, self.tp.rank, self.tp.size)
                lin.out_shape = tuple(lin.kernel.shape[len(lin.in_shape):])
                lin.in_shape = tuple(lin.kernel.shape[:len(lin.in_shape)])

    def forward(self, x: torch.Tensor, positions: torch.Tensor | None, mask: torch.Tensor | None = None,
                default_positions: bool = False) -> torch.Tensor:
        tp = self.tp
        if tp is not None:
            # token-sharded input [1, T/t, D]: gather the group's tokens, attend with the local heads over the full
            # sequences, scatter the output projection's partial sums back to the token shards
            from mintext_b200.parallel import tp as tpm

            if mask is not None:
                raise NotImplementedError("explicit attention masks are not supported under tensor parallelism")
            B, S = tp.batch_shape
            Tl, D = x.shape[-2], x.shape[-1]
            x = tpm.all_gather_tokens(x.reshape(Tl, D), tp).view(B, S, D)
            if positions is None or positions.shape[-1] != S:
                positions = torch.arange(S, device=x.device)[None].expand(B, -1)
        B, S, _ = x.shape
        H = self.local_heads
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
        y = self.out(o)
        if tp is not None:
            from mintext_b200.parallel import tp as tpm

            return tpm.reduce_scatter_tokens(y.reshape(B * S, -1), tp).view(1, -1, y.shape[-1])
        return y
