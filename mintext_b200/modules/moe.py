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
        logits = self.gate(x)
        if self.router_type == "softmax_topk":
            idx, w, probs, aux = oracle.router_softmax_topk(logits, self.num_experts_per_tok, self.norm_topk_prob)
            self.last_aux_loss = aux
            return idx, w, probs
        self.last_aux_loss = None
        return oracle.router_sigmoid_group(
            logits, self.e_score_correction_bias, self.num_experts_per_tok, self.n_group, self.topk_group,
            self.norm_topk_prob, self.routed_scaling_factor)


class MoEExperts(nn.Module):
    def __init__(self, config, *, rngs=None):
        super().__init__()
        E, D, I = config.num_experts, config.hidden_size, config.moe_intermediate_size
        self.num_experts = E
        self.dtype = config.torch_dtype
        self.act_name = config.hidden_activation
        wdt = config.torch_weight_dtype
        # the reference's initialiser divides by total // shape[2], i.e. E*D and E*I: the std shrinks with E
        self.gate_up_proj = nn.Parameter(truncated_normal_init((E, D, 2 * I), E * D, rngs, wdt))
        self.gate_up_proj.logical_axes = ("exp", "embed", "mlp")
        self.down_proj = nn.Parameter(truncated_normal_init((E, I, D), E * I, rngs, wdt))
        self.down_proj.logical_axes = ("exp", "mlp", "embed")

    def forward(self, x: torch.Tensor, topk_indices: torch.Tensor, topk_weights: torch.Tensor) -> torch.Tensor:
        """x ``[N,D]`` -> ``[N,D]``: route, grouped GEMM, SwiGLU on the column halves, grouped GEMM, unroute."""
        from mintext_b200.ops import moe as moe_ops

        gu = self.gate_up_proj if self.gate_up_proj.dtype == self.dtype else self.gate_up_proj.to(self.dtype)
        dn = self.down_proj if self.down_proj.dtype == self.dtype else self.down_proj.to(self.dtype)
        if moe_ops.cuda_path(x) and gu is self.gate_up_proj:
            return moe_ops.experts_forward(x, topk_indices, topk_weights, gu, dn, self.act_name)
        rows, sort_idx, sizes = kernels.route(x, topk_indices, self.num_experts)
        h = kernels.grouped_matmul_vjp(rows, gu, sizes)
        h = F.gated_act(h, self.act_name)
        y = kernels.grouped_matmul_vjp(h, dn, sizes)
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
