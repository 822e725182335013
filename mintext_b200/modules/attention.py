"""Multi-head / grouped-query attention with RoPE, optional QK-norm, sliding window, logit soft-capping and
sigmoid output gating (reference: mintext/modules/attention.py).

Projection kernels keep the reference shapes (``query [D,H,dh]`` or ``[D,H,2dh]`` when gated, ``key``/``value``
``[D,Hkv,dh]``, ``out [H,dh,D]``).  The attention core is one call into :func:`ops.functional.attention`, which
runs the flash kernel on CUDA and the fp32-softmax oracle elsewhere; causal and window masks are never
materialised on the kernel path.
"""

from __future__ import annotations

import torch
from torch import nn

from mintext_b200.ops import functional as F
from mintext_b200.ops.oracle import sliding_window_mask

from .linear import Linear
from .norm import RMSNorm
from .rope import RotaryEmbedding


def make_sliding_window_mask(seq_len: int, window_size: int, dtype=torch.float32) -> torch.Tensor:
    """Additive ``[1,1,S,S]`` mask that keeps ``0 <= i - j < window_size``."""
    return sliding_window_mask(seq_len, window_size, dtype)


class Attention(nn.Module):
    def __init__(self, config, *, rngs=None, mesh=None, use_qk_norm: bool = False, sliding_window: int | None = None,
                 use_gate: bool = False, rope_local_theta: float | None = None):
        super().__init__()
        self.num_attention_heads = config.num_attention_heads
        self.num_key_value_heads = config.num_key_value_heads
        self.head_dim = config.head_dim
        self.dtype = config.torch_dtype
        self.use_qk_norm = use_qk_norm
        self.sliding_window = sliding_window
        self.use_gate = use_gate
        self.attn_logit_softcapping = config.attn_logit_softcapping
        D, H, Hkv, dh = config.hidden_size, config.num_attention_heads, config.num_key_value_heads, config.head_dim
        wdt = config.torch_weight_dtype
        from mintext_b200.parallel.tp import current_tp

        self.tp = current_tp() if (current_tp() is not None and current_tp().size > 1) else None
        qps = config.query_pre_attn_scalar
        self.scale = (qps if qps is not None else dh) ** -0.5
        q_dim = 2 * dh if use_gate else dh
        self.query = Linear(D, (H, q_dim), self.dtype, wdt, ("embed", "heads", "kv"), rngs=rngs, name="query_proj")
        self.key = Linear(D, (Hkv, dh), self.dtype, wdt, ("embed", "kv_heads", "kv"), rngs=rngs, name="key_proj")
        self.value = Linear(D, (Hkv, dh), self.dtype, wdt, ("embed", "kv_heads", "kv"), rngs=rngs, name="value_proj")
        self.out = Linear((H, dh), D, self.dtype, wdt, ("heads", "kv", "embed"), rngs=rngs, name="out_proj")
        self.rope = RotaryEmbedding(config, theta=rope_local_theta)
        if use_qk_norm:
            self.q_norm = RMSNorm(dh, config.rms_norm_eps, self.dtype)
            self.k_norm = RMSNorm(dh, config.rms_norm_eps, self.dtype)
        if self.tp is not None:
            # keep this rank's heads: the full kernels were drawn from the model's stream, so the slices equal
            # the corresponding heads of the unsharded model
            qlo, qhi = self.tp.shard(H, "num_attention_heads")
            klo, khi = self.tp.shard(Hkv, "num_key_value_heads")
            for lin, (a, b), dim in ((self.query, (qlo, qhi), 1), (self.key, (klo, khi), 1),
                                     (self.value, (klo, khi), 1), (self.out, (qlo, qhi), 0)):
                full = lin.kernel.data
                lin.kernel = nn.Parameter((full[:, a:b] if dim == 1 else full[a:b]).clone().contiguous())
                lin.kernel.logical_axes = ("embed", "heads", "kv") if dim == 1 else ("heads", "kv", "embed")
                lin.kernel.tensor_parallel = True
                lin.kernel.shard_spec = (dim, self.tp.rank, self.tp.size)
            self.local_heads, self.local_kv_heads = qhi - qlo, khi - klo

    def _forward_tp(self, x, positions, default_positions):
        """Token-sharded input ``[1, T/t, D]``: gather tokens into the q/k/v projections of the local heads,
        attend over the full sequences, scatter the output projection's partial sums back to token shards."""
        from mintext_b200.parallel import tp as tpm

        tp = self.tp
        B, S = tp.batch_shape
        Tl, D = x.shape[-2], x.shape[-1]
        Hl, Hk, dh = self.local_heads, self.local_kv_heads, self.head_dim
        qd = 2 * dh if self.use_gate else dh
        _, (q_raw, k, v) = tpm.column_linear(
            x.reshape(Tl, D), [tpm.as_matrix(self.query.kernel, D), tpm.as_matrix(self.key.kernel, D),
                               tpm.as_matrix(self.value.kernel, D)], tp, self.dtype)
        q_raw, k, v = q_raw.view(B, S, Hl, qd), k.view(B, S, Hk, dh), v.view(B, S, Hk, dh)
        q, gate = (q_raw.chunk(2, dim=-1) if self.use_gate else (q_raw, None))
        if self.use_qk_norm:
            q, k = self.q_norm(q.contiguous()), self.k_norm(k)
        if positions is None or positions.shape[-1] != S:
            positions = torch.arange(S, device=x.device)[None].expand(B, -1)
        q = self.rope(q, positions, default_positions)
        k = self.rope(k, positions, default_positions)
        o = F.attention(q, k, v, self.scale, causal=True, window=self.sliding_window,
                        softcap=self.attn_logit_softcapping)
        if gate is not None:
            o = F.gate_mul(o, gate, "sigmoid")
        y = tpm.row_linear(o.reshape(B * S, Hl * dh), tpm.as_matrix(self.out.kernel, Hl * dh), tp, self.dtype)
        return y.view(1, Tl, D)

    def forward(self, x: torch.Tensor, positions: torch.Tensor | None, mask: torch.Tensor | None = None,
                default_positions: bool = False) -> torch.Tensor:
        if self.tp is not None:
            if mask is not None:
                raise NotImplementedError("explicit attention masks are not supported under tensor parallelism")
            return self._forward_tp(x, positions, default_positions)
        q_raw = self.query(x)
        k = self.key(x)
        v = self.value(x)
        if self.use_gate:
            q, gate = q_raw.chunk(2, dim=-1)
        else:
            q, gate = q_raw, None
        if self.use_qk_norm:
            q = self.q_norm(q.contiguous())
            k = self.k_norm(k)
        q = self.rope(q, positions, default_positions)
        k = self.rope(k, positions, default_positions)
        # an explicit additive mask already encodes causality (and the caller's choice of window)
        if mask is not None:
            m = mask
            if self.sliding_window is not None:
                m = m + sliding_window_mask(x.shape[1], self.sliding_window, device=x.device).to(m.dtype)
            o = F.attention(q, k, v, self.scale, causal=False, window=None, softcap=self.attn_logit_softcapping,
                            mask=m)
        else:
            o = F.attention(q, k, v, self.scale, causal=True, window=self.sliding_window,
                            softcap=self.attn_logit_softcapping)
        o = F.checkpoint_name(o, "context")
        if gate is not None:
            o = F.gate_mul(o, gate, "sigmoid")
        return self.out(o)
