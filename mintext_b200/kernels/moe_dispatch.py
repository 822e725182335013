"""Token dispatch for capacity-free, drop-free MoE (reference: mintext/kernels/moe_dispatch.py).

``route`` orders the ``N*K`` (token, slot) rows by expert with a stable counting sort so each expert's rows are
contiguous; ``unroute`` applies the inverse permutation and the weighted sum over the K slots.  Both are
differentiable: the backward of the row permutation is the inverse gather, the backward of the weighted sum
gives gradients to the expert outputs and to the routing weights.
"""

from __future__ import annotations

import torch

from mintext_b200.ops import oracle


def route(tokens: torch.Tensor, topk_indices: torch.Tensor, num_experts: int):
    """tokens ``[N,D]``, topk_indices ``[N,K]`` -> (sorted ``[N*K,D]``, sort_indices ``[N*K]``, group_sizes ``[E]``)."""
    from mintext_b200.ops import moe as moe_ops

    if moe_ops.cuda_path(tokens):
        return moe_ops.route_cuda(tokens, topk_indices, num_experts)
    return oracle.route(tokens, topk_indices, num_experts)


def unroute(sorted_output: torch.Tensor, sort_indices: torch.Tensor, topk_weights: torch.Tensor,
            num_experts_per_tok: int) -> torch.Tensor:
    """sorted_output ``[N*K,D]`` -> ``[N,D]`` = ``sum_k w[n,k] * y[n,k]``."""
    from mintext_b200.ops import moe as moe_ops

    if moe_ops.cuda_path(sorted_output):
        return moe_ops.unroute_cuda(sorted_output, sort_indices, topk_weights, num_experts_per_tok)
    return oracle.unroute(sorted_output, sort_indices, topk_weights, num_experts_per_tok)
