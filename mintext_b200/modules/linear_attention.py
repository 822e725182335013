"""Gated Delta Rule linear attention (Qwen3-Next GDN; reference: mintext/modules/linear_attention.py)."""

from __future__ import annotations

import torch
from torch import nn

from mintext_b200.ops import functional as F
from mintext_b200.ops import oracle

from .linear import Linear
from .norm import RMSNorm


def chunk_gated_delta_rule(q, k, v, beta, g, chunk_size: int = 64):
    """q,k ``[B,H,S,dk]``, v ``[B,H,S,dv]``, beta,g ``[B,H,S]`` -> ``[B,H,S,dv]`` (fp32)."""
    from mintext_b200.ops import gdn

    if gdn.cuda_path(q, v, chunk_size):
        return gdn.chunk_gated_delta_rule_cuda(q, k, v, beta, g, chunk_size)
    return oracle.chunk_gated_delta_rule(q, k, v, beta, g, chunk_size)


class GatedDeltaRuleAttention(nn.Module):
    def __init__(self, config, *, rngs=None):
        super().__init__()
        self.dtype = dt = config.torch_dtype
        wdt = config.torch_weight_dtype
        D = config.hidden_size
        self.num_k_heads = Hk = config.linear_num_key_heads or config.num_attention_heads
        self.num_v_heads = Hv = config.linear_num_value_heads or config.num_attention_heads
        self.key_head_dim = dk = config.linear_key_head_dim
        self.value_head_dim = dv = config.linear_value_head_dim
        self.v_heads_per_k_group = Hv // Hk
        self.chunk_size = 64
        key_dim, value_dim = Hk * dk, Hv * dv
        conv_dim = 2 * key_dim + value_dim
        self.in_proj_qkvz = Linear(D, 2 * key_dim + 2 * value_dim, dt, wdt, ("embed", "mlp"), rngs=rngs)
        self.in_proj_ba = Linear(D, 2 * Hv, dt, wdt, ("embed", "mlp"), rngs=rngs)
        ksz = config.linear_conv_kernel_dim
        self.conv_weight = nn.Parameter((torch.randn(conv_dim, 1, ksz, generator=rngs) * 0.02).to(wdt))
        self.conv_weight.logical_axes = (None, None, None)
        self.A_log = nn.Parameter(torch.log(0.5 + torch.rand(Hv, generator=rngs) * 15.5))
        self.A_log.logical_axes = (None,)
        self.dt_bias = nn.Parameter(torch.ones(Hv))
        self.dt_bias.logical_axes = (None,)
        self.norm = RMSNorm(dv, config.rms_norm_eps, dt)
        self.out_proj = Linear(value_dim, D, dt, wdt, ("mlp", "embed"), rngs=rngs)
        # Tensor parallelism: key heads (with their value-head groups) are split over the group.  The two input
        # projections are column-parallel in the grouped per-key-head layout, the output projection row-parallel; the
        # depth-wise conv weights, A_log, dt_bias and the output norm stay whole on every rank, which uses the rows of
        # its own heads - its gradient for them is a partial sum that the engine's cross-rank gradient sum completes.
        from mintext_b200.parallel.tp import current_tp

        self.tp = current_tp() if (current_tp() is not None and current_tp().size > 1) else None
        self.k_head_lo, self.local_k_heads = 0, Hk
        if self.tp is not None:
            lo, hi = self.tp.shard(Hk, "linear_num_key_heads")
            self.k_head_lo, self.local_k_heads = lo, hi - lo
            g = self.v_heads_per_k_group
            per_qkvz, per_ba, per_out = 2 * dk + 2 * g * dv, 2 * g, g * dv
            for lin, dim, per in ((self.in_proj_qkvz, 1, per_qkvz), (self.in_proj_ba, 1, per_ba), (self.out_proj, 0, per_out)):
                full = lin.kernel.data
                axes = lin.kernel.logical_axes
                a, b = lo * per, hi * per
                lin.kernel = nn.Parameter((full[:, a:b] if dim == 1 else full[a:b]).clone().contiguous())
                lin.kernel.logical_axes = axes
                lin.kernel.tensor_parallel = True
                lin.kernel.shard_spec = (dim, self.tp.rank, self.tp.size)
                lin.out_shape = tuple(lin.kernel.shape[len(lin.in_shape):])
                lin.in_shape = tuple(lin.kernel.shape[:len(lin.in_shape)])

    def _split_qkvz(self, qkvz: torch.Tensor):
        """HF grouped layout: per key head ``[q(dk) | k(dk) | v(g*dv) | z(g*dv)]`` (this rank's key heads)."""
        B, S, _ = qkvz.shape
        Hk, Hv = self.local_k_heads, self.local_k_heads * self.v_heads_per_k_group
        vg = self.v_heads_per_k_group * self.value_head_dim
        grouped = qkvz.reshape(B, S, Hk, 2 * self.key_head_dim + 2 * vg)
        q, k, v, z = grouped.split([self.key_head_dim, self.key_head_dim, vg, vg], dim=-1)
        v = v.reshape(B, S, Hv, self.value_head_dim)
        z = z.reshape(B, S, Hv, self.value_head_dim)
        return q, k, v, z

    def _split_ba(self, ba: torch.Tensor):
        B, S, _ = ba.shape
        g = self.v_heads_per_k_group
        grouped = ba.reshape(B, S, self.local_k_heads, 2 * g)
        b, a = grouped.split([g, g], dim=-1)
        Hv = self.local_k_heads * g
        return b.reshape(B, S, Hv), a.reshape(B, S, Hv)

    def _local_head_params(self):
        """Conv weights, A_log and dt_bias of this rank's heads (all of them without tensor parallelism)."""
        if self.tp is None:
            return self.conv_weight, self.A_log, self.dt_bias
        g, dk, dv = self.v_heads_per_k_group, self.key_head_dim, self.value_head_dim
        lo, hi = self.k_head_lo, self.k_head_lo + self.local_k_heads
        key_total = self.num_k_heads * dk
        cw = self.conv_weight
        conv = torch.cat([cw[lo * dk:hi * dk], cw[key_total + lo * dk:key_total + hi * dk],
                          cw[2 * key_total + lo * g * dv:2 * key_total + hi * g * dv]], dim=0)
        return conv, self.A_log[lo * g:hi * g], self.dt_bias[lo * g:hi * g]

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        tp = self.tp
        if tp is not None:
            # token-sharded input [1, T/t, D]: gather the group's tokens, run this rank's heads over the full
            # sequences, scatter the output projection's partial sums back to the token shards
            from mintext_b200.parallel import tp as tpm

            B, S = tp.batch_shape
            x = tpm.all_gather_tokens(x.reshape(-1, x.shape[-1]), tp).view(B, S, x.shape[-1])
        B, S, _ = x.shape
        Hk, Hv = self.local_k_heads, self.local_k_heads * self.v_heads_per_k_group
        conv_weight, A_log, dt_bias = self._local_head_params()
        q, k, v, z = self._split_qkvz(self.in_proj_qkvz(x))
        b_raw, a = self._split_ba(self.in_proj_ba(x))
        beta = torch.sigmoid(b_raw.float())
        key_total = Hk * self.key_head_dim
        value_total = Hv * self.value_head_dim
        qkv = torch.cat([q.reshape(B, S, key_total), k.reshape(B, S, key_total), v.reshape(B, S, value_total)], dim=-1)
        qkv = F.causal_conv1d_silu(qkv, conv_weight if conv_weight.dtype == self.dtype else conv_weight.to(self.dtype))
        qc, kc, vc = qkv.split([key_total, key_total, value_total], dim=-1)
        qh = qc.reshape(B, S, Hk, self.key_head_dim)
        kh = kc.reshape(B, S, Hk, self.key_head_dim)
        vh = vc.reshape(B, S, Hv, self.value_head_dim)
        g = -torch.exp(A_log.float()) * torch.nn.functional.softplus(a.float() + dt_bias.float())
        if self.v_heads_per_k_group > 1:
            qh = qh.repeat_interleave(self.v_heads_per_k_group, dim=2)
            kh = kh.repeat_interleave(self.v_heads_per_k_group, dim=2)
        out = chunk_gated_delta_rule(
            qh.float().transpose(1, 2), kh.float().transpose(1, 2), vh.float().transpose(1, 2),
            beta.transpose(1, 2), g.transpose(1, 2), chunk_size=self.chunk_size)
        out = out.transpose(1, 2).to(self.dtype)
        out = F.gate_mul(self.norm(out.contiguous()), z.to(self.dtype), "silu")
        y = self.out_proj(out.reshape(B, S, value_total))
        if tp is not None:
            from mintext_b200.parallel import tp as tpm

            return tpm.reduce_scatter_tokens(y.reshape(B * S, -1), tp).view(1, -1, y.shape[-1])
        return y
