"""Mixture-of-experts block: router, routed experts, optional shared expert (reference: mintext/modules/moe.py).

Two routers: the DeepSeek-V3 sigmoid / group-limited top-k router with a load-balancing selection bias (the
reference's only router) and a softmax top-k router with the Switch-style auxiliary loss (Qwen3-MoE).
Experts hold the fused ``gate_up_proj [E, D, 2I]`` (gate = first I columns) and ``down_proj [E, I, D]``.
"""

from __future__ import annotations

import torch
from torch import nn

from mintext_b200 import kernels
from mintext_b200.ops import functional as F
from mintext_b200.ops import oracle

from .linear import MLP, Linear, truncated_normal_init


class MoERouter(nn.Module):
    def __init__(self, config, *, rngs=None):
        super().__init__()
        self.num_experts = config.num_experts
        self.num_experts_per_tok = config.num_experts_per_tok
        self.n_group = config.n_group
        self.topk_group = config.topk_group
        self.norm_topk_prob = config.norm_topk_prob
        self.routed_scaling_factor = config.routed_scaling_factor
        self.router_type = config.router_type
        self.gate = Linear(config.hidden_size, config.num_experts, config.torch_dtype, config.torch_weight_dtype,
                           ("embed", "mlp"), rngs=rngs)
        # selection-only bias for loss-free balancing: no gradient, no weight decay, updated out of band
        self.e_score_correction_bias = nn.Parameter(torch.zeros(config.num_experts, dtype=torch.float32),
                                                    requires_grad=False)
        self.e_score_correction_bias.logical_axes = (None,)
        self.last_aux_loss: torch.Tensor | None = None

    def forward(self, x: torch.Tensor):
        """x ``[N, D]`` -> (topk_indices ``[N,K]``, topk_weights ``[N,K]`` fp32, scores ``[N,E]`` fp32)."""
        from mintext_b200.ops import moe as moe_ops

        logits = self.gate(x)
        impl = moe_ops if moe_ops.router_cuda_path(logits, self.num_experts, self.num_experts_per_tok,
                                                   self.n_group) else oracle
        if self.router_type == "softmax_topk":
            idx, w, probs, aux = impl.router_softmax_topk(logits, self.num_experts_per_tok, self.norm_topk_prob)
            from mintext_b200.parallel.tp import current_tp

            tp = current_tp()
            if tp is not None and tp.size > 1:
                # Token-sharded activations: this rank routed its own share of the group's tokens.  With the
                # assignment fractions f_e taken over the whole group (a small all-reduce of counts, no gradient) and
                # the mean probabilities P_e over the rank's tokens, the mean of the ranks' terms is exactly the
                # auxiliary loss E * sum_e f_e P_e of the group's batch.
                import torch.distributed as dist

                N, E = probs.shape
                counts = oracle.histogram(idx, E).float()
                dist.all_reduce(counts, group=tp.group)
                f = counts / (N * tp.size * self.num_experts_per_tok)
                aux = E * (f * probs.mean(0)).sum()
            self.last_aux_loss = aux
            return idx, w, probs
        self.last_aux_loss = None
        return impl.router_sigmoid_group(
            logits, self.e_score_correction_bias, self.num_experts_per_tok, self.n_group, self.topk_group,
            self.norm_topk_prob, self.routed_scaling_factor)


def _per_expert_init(shape_tail, fan_in, lo, hi, rngs, dtype):
    """Experts ``lo .. hi`` of a stacked parameter, each drawn from its own generator (seeded from one value taken
    off the model's stream), so that a rank holding only a slice of the experts initialises exactly the values the
    unsharded model would have there."""
    tag = int(torch.randint(0, 2 ** 31 - 1, (1,), generator=rngs))
    out = None
    for e in range(lo, hi):
        g = torch.Generator().manual_seed((tag + 104729 * e) % (2 ** 63 - 1))
        w = truncated_normal_init(shape_tail, fan_in, g, dtype)
        if out is None:  # on whichever device the initialiser draws
            out = torch.empty((hi - lo,) + tuple(shape_tail), dtype=dtype, device=w.device)
        out[e - lo] = w
    return out


class MoEExperts(nn.Module):
    """Routed experts.  Under expert parallelism (a process-wide :class:`ExpertParallel` context) the module holds
    only this rank's ``E / ep`` experts and exchanges tokens with the other ranks."""

    def __init__(self, config, *, rngs=None):
        super().__init__()
        from mintext_b200.parallel.ep import current_ep

        E, D, I = config.num_experts, config.hidden_size, config.moe_intermediate_size
        self.num_experts = E
        self.dtype = config.torch_dtype
        self.act_name = config.hidden_activation
        # grouped-GEMM tilings per projection: from the config, or set later by the autotuner (train.py)
        self.gate_up_tiling = tuple(config.moe_gate_up_tiling) or None
        self.down_tiling = tuple(config.moe_down_tiling) or None
        self.use_fp8 = bool(config.moe_use_fp8)  # expert GEMMs (forward, data gradient) in block-scaled FP8
        self.ep = current_ep()
        lo, hi = self.ep.local_expert_range(E) if self.ep is not None else (0, E)
        self.local_range = (lo, hi)
        wdt = config.torch_weight_dtype
        rngs = rngs if rngs is not None else torch.Generator().manual_seed(0)
        # the reference's initialiser divides by total // shape[2], i.e. E*D and E*I: the std shrinks with E
        self.gate_up_proj = nn.Parameter(_per_expert_init((D, 2 * I), E * D, lo, hi, rngs, wdt))
        self.gate_up_proj.logical_axes = ("exp", "embed", "mlp")
        self.down_proj = nn.Parameter(_per_expert_init((I, D), E * I, lo, hi, rngs, wdt))
        self.down_proj.logical_axes = ("exp", "mlp", "embed")
        if self.ep is not None and self.ep.size > 1:
            self.gate_up_proj.expert_parallel = True
            self.down_proj.expert_parallel = True
            self.gate_up_proj.shard_spec = self.down_proj.shard_spec = (0, self.ep.rank, self.ep.size)

    def forward(self, x: torch.Tensor, topk_indices: torch.Tensor, topk_weights: torch.Tensor) -> torch.Tensor:
        """x ``[N,D]`` -> ``[N,D]``: route, grouped GEMM, SwiGLU on the column halves, grouped GEMM, unroute."""
        from mintext_b200.ops import moe as moe_ops

        gu = self.gate_up_proj if self.gate_up_proj.dtype == self.dtype else self.gate_up_proj.to(self.dtype)
        dn = self.down_proj if self.down_proj.dtype == self.dtype else self.down_proj.to(self.dtype)
        if self.ep is not None and self.ep.size > 1:
            from mintext_b200.parallel import ep as ep_mod

            if self.ep.fused and moe_ops.cuda_path(x) and gu is self.gate_up_proj:
                return ep_mod.experts_forward_peer(self.ep, x, topk_indices, topk_weights, gu, dn, self.act_name,
                                                   self.num_experts, fp8=self.use_fp8)
            return ep_mod.experts_forward_collective(self.ep, x, topk_indices, topk_weights, self.gate_up_proj,
                                                     self.down_proj, self.act_name, self.num_experts, self.dtype)
        if moe_ops.cuda_path(x) and gu is self.gate_up_proj:
            return moe_ops.experts_forward(x, topk_indices, topk_weights, gu, dn, self.act_name, self.gate_up_tiling,
                                           self.down_tiling, self.use_fp8)
        rows, sort_idx, sizes = kernels.route(x, topk_indices, self.num_experts)
        h = kernels.grouped_matmul_vjp(rows, gu, sizes, tiling=self.gate_up_tiling)
        h = F.gated_act(h, self.act_name)
        y = kernels.grouped_matmul_vjp(h, dn, sizes, tiling=self.down_tiling)
        return kernels.unroute(y, sort_idx, topk_weights, topk_indices.shape[1])


class MoEBlock(nn.Module):
    """Returns ``(output [B,S,D], aux)`` with ``aux = {"topk_indices", "scores"[, "aux_loss"]}``."""

    def __init__(self, config, *, rngs=None):
        super().__init__()
        self.router = MoERouter(config, rngs=rngs)
        self.experts = MoEExperts(config, rngs=rngs)
        self.n_shared_experts = config.n_shared_experts
        if config.n_shared_experts > 0:
            self.shared_expert = MLP(config, rngs=rngs,
                                     intermediate_size=config.moe_intermediate_size * config.n_shared_experts)
        else:
            self.shared_expert = None
        if self.shared_expert is not None and config.shared_expert_gate:
            self.shared_expert_gate = Linear(config.hidden_size, 1, config.torch_dtype, config.torch_weight_dtype,
                                             ("embed", None), rngs=rngs)
        else:
            self.shared_expert_gate = None

    def forward(self, x: torch.Tensor):
        B, S, D = x.shape
        flat = x.reshape(B * S, D)
        idx, w, scores = self.router(flat)
        out = self.experts(flat, idx, w).reshape(B, S, D)
        if self.shared_expert is not None:
            shared = self.shared_expert(x)
            if self.shared_expert_gate is not None:
                shared = shared * torch.sigmoid(self.shared_expert_gate(x))
            out = out + shared
        aux = {"topk_indices": idx, "scores": scores}
        if self.router.last_aux_loss is not None:
            aux["aux_loss"] = self.router.last_aux_loss
        return out, aux
