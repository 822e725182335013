"""Gradient accumulation over micro-batches (reference: mintext/optim/grad_accumulation.py).

The batch dimension of every entry of ``data`` is split into ``num_micro_steps`` equal parts; gradients and
losses are averaged; the auxiliary output of the last micro-batch is returned.
"""

from __future__ import annotations

from typing import Callable

import torch


def accumulate_gradients(loss_fn: Callable, params: dict[str, torch.Tensor], data: dict[str, torch.Tensor],
                         num_micro_steps: int):
    """``loss_fn(params, micro_batch) -> (loss, aux)``.  Returns ``(mean_loss, last_aux, mean_grads)``."""
    names = list(params)
    tensors = [params[n] for n in names]
    B = next(iter(data.values())).shape[0]
    if B % num_micro_steps != 0:
        raise ValueError(f"batch size {B} is not divisible by num_micro_steps {num_micro_steps}")
    mb = B // num_micro_steps
    total_loss = None
    sums: list[torch.Tensor | None] = [None] * len(tensors)
    aux = None
    for i in range(num_micro_steps):
        micro = {k: v[i * mb:(i + 1) * mb] for k, v in data.items()}
        loss, aux = loss_fn(params, micro)
        grads = torch.autograd.grad(loss, tensors, allow_unused=True)
        total_loss = loss.detach() if total_loss is None else total_loss + loss.detach()
        for j, g in enumerate(grads):
            if g is not None:
                sums[j] = g if sums[j] is None else sums[j] + g
    mean_grads = {n: (s / num_micro_steps if s is not None else None) for n, s in zip(names, sums)}
    return total_loss / num_micro_steps, aux, mean_grads
