"""Learning-rate schedules and the AdamW / Muon optimizers (reference: mintext/optim/optimizer.py, which wires
optax; the update rules are restated here).

``create_optimizer(config)`` returns an :class:`Optimizer` with optax-like ``init`` / ``update`` semantics over a
``{name: tensor}`` dict.  This per-tensor implementation is the semantic reference (and the CPU path); on a GPU
the training engine runs the same AdamW rule as one fused kernel over flat fp32 shards.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Callable

import torch

from mintext_b200.ops import oracle


# ------------------------------------------------------------------------------------------ schedules
def create_lr_schedule(config) -> Callable[[int], float]:
    """Linear warm-up from 0 over ``max(int(steps * warmup_fraction), 1)`` steps, then cosine / linear decay to
    ``lr * lr_final_fraction``, or warm-up / stable / decay (WSD) with a linear or cosine tail."""
    peak = float(config.learning_rate)
    total = int(config.steps)
    warm = max(int(total * config.warmup_steps_fraction), 1)
    final = peak * float(config.lr_final_fraction)
    kind = config.lr_schedule

    def warmup(step: int) -> float:
        return peak * step / warm

    if kind == "cosine":
        decay = max(total - warm, 1)
        alpha = float(config.lr_final_fraction)

        def sched(step: int) -> float:
            if step < warm:
                return warmup(step)
            t = min(step - warm, decay)
            return peak * (alpha + (1 - alpha) * 0.5 * (1 + math.cos(math.pi * t / decay)))

        return sched
    if kind == "linear":
        decay = max(total - warm, 1)

        def sched(step: int) -> float:
            if step < warm:
                return warmup(step)
            t = min(step - warm, decay)
            return peak + (final - peak) * t / decay

        return sched
    if kind == "wsd":
        tail = max(int(total * config.wsd_decay_steps_fraction), 1)
        stable = max(total - warm - tail, 0)
        style = config.wsd_decay_style

        def sched(step: int) -> float:
            if step < warm:
                return warmup(step)
            if step < warm + stable:
                return peak
            t = min(step - warm - stable, tail)
            if style == "cosine":
                alpha = float(config.lr_final_fraction)
                return peak * (alpha + (1 - alpha) * 0.5 * (1 + math.cos(math.pi * t / tail)))
            return peak + (final - peak) * t / tail

        return sched
    raise ValueError(f"Unknown lr_schedule: {kind}")


# ------------------------------------------------------------------------------------------ helpers
def weight_decay_mask(name: str) -> bool:
    """Every parameter is decayed except the router's selection bias (norm scales and embeddings are decayed
    too, as in the reference: mintext/optim/optimizer.py:82-89)."""
    return "e_score_correction_bias" not in name


def muon_matrix_view(name: str, shape: tuple[int, ...]) -> tuple[int, int, int] | None:
    """How Muon sees a parameter: ``(batch, rows, cols)`` of the matrices to orthogonalise, or None when the
    parameter is handled by Adam (1-D, embeddings, norm scales, router bias).  Mirrors the dimension numbers of
    mintext/optim/optimizer.py:92-114: 2-D kernels are (in, out); q/k/v-style 3-D kernels ``[D,H,dh]`` reduce
    over D with outputs (H, dh); the attention ``out`` kernel ``[H,dh,D]`` reduces over (H, dh); expert stacks
    ``[E,in,out]`` are a batch of E matrices."""
    if "token_embedder" in name or name.endswith("scale") or "e_score_correction_bias" in name or len(shape) < 2:
        return None
    if "conv_weight" in name:
        return None
    if len(shape) == 2:
        return (1, shape[0], shape[1])
    if len(shape) == 3:
        if "experts" in name or name.endswith("gate_up_proj") or name.endswith("down_proj"):
            return (shape[0], shape[1], shape[2])
        if ".out." in name or name.endswith("out.kernel"):
            return (1, shape[0] * shape[1], shape[2])
        return (1, shape[0], shape[1] * shape[2])
    return None


def muon_slice_axis(name: str, param) -> int | None:
    """For a parameter of which a tensor-parallel rank holds a slice: which dimension of its Muon matrix view is
    sliced (-2 rows, -1 columns); None for whole matrices (expert stacks are whole matrices per expert)."""
    spec = getattr(param, "shard_spec", None)
    if spec is None or not getattr(param, "tensor_parallel", False) or int(spec[2]) < 2:
        return None
    shape = tuple(param.shape)
    if muon_matrix_view(name, shape) is None:
        return None
    dim = int(spec[0])
    if len(shape) == 2:
        return -2 if dim == 0 else -1
    if "experts" in name or name.endswith("gate_up_proj") or name.endswith("down_proj"):
        return None if dim == 0 else (-2 if dim == 1 else -1)
    if ".out." in name or name.endswith("out.kernel"):
        return -2 if dim in (0, 1) else -1
    return -2 if dim == 0 else -1


def muon_sliced_update(mu_hat: torch.Tensor, view: tuple[int, int, int], axis: int, group, steps: int, eps: float,
                       consistent_rms: float | None):
    """Orthogonalised update of a sliced matrix and its shape factor (that of the whole matrix)."""
    import torch.distributed as dist

    from mintext_b200.ops import oracle

    b, r, c = view
    n = dist.get_world_size(group)
    upd = oracle.newton_schulz_sliced(mu_hat.reshape(b, r, c).float(), axis,
                                      lambda t: dist.all_reduce(t, group=group), steps, eps)
    full = (r * n, c) if axis == -2 else (r, c * n)
    return upd, muon_shape_scale(full[0], full[1], consistent_rms)


def muon_shape_scale(fan_in: int, fan_out: int, consistent_rms: float | None = None) -> float:
    """Factor applied to an orthogonalised ``[fan_in, fan_out]`` update: ``sqrt(max(1, fan_out / fan_in))`` (the
    update of a matrix that widens its input is scaled up, one that narrows it is left alone), or
    ``consistent_rms * sqrt(max(fan_in, fan_out))`` when a target RMS is configured.  The reference gets this from
    ``optax.contrib.muon`` with the reduction axis first and the output axis last
    (mintext/optim/optimizer.py:92-150)."""
    if consistent_rms is not None:
        return math.sqrt(max(fan_in, fan_out)) * float(consistent_rms)
    return math.sqrt(max(1.0, fan_out / fan_in))


def global_norm(tensors) -> torch.Tensor:
    ts = [t for t in tensors if t is not None]
    if not ts:
        return torch.zeros(())
    return torch.sqrt(sum((t.float() ** 2).sum() for t in ts))


@dataclass
class OptState:
    count: int = 0
    mu: dict = field(default_factory=dict)
    nu: dict = field(default_factory=dict)


class Optimizer:
    """``clip_by_global_norm(threshold) -> adamw | muon`` over a dict of tensors."""

    def __init__(self, config):
        self.config = config
        self.kind = config.optimizer
        self.schedule = create_lr_schedule(config)
        self.clip = float(config.gradient_clip_threshold)

    def init(self, params: dict[str, torch.Tensor]) -> OptState:
        st = OptState()
        for n, p in params.items():
            st.mu[n] = torch.zeros_like(p, dtype=torch.float32)
            if self.kind == "adamw" or muon_matrix_view(n, tuple(p.shape)) is None:
                st.nu[n] = torch.zeros_like(p, dtype=torch.float32)
        return st

    @torch.no_grad()
    def update(self, params: dict[str, torch.Tensor], grads: dict[str, torch.Tensor], state: OptState,
               step: int, grad_norm: float | None = None) -> None:
        """In-place update of ``params`` for schedule position ``step`` (the pre-increment step counter).
        ``grad_norm``: the norm to clip by when it is not that of ``grads`` alone (a multi-process run, where a rank
        holds slices of some gradients)."""
        cfg = self.config
        lr = self.schedule(step)
        if self.clip > 0:
            gn = float(grad_norm) if grad_norm is not None else float(global_norm(grads.values()))
            factor = self.clip / max(gn, self.clip)  # optax.clip_by_global_norm
        else:
            factor = 1.0
        state.count += 1
        t = state.count
        tp_group = None
        if self.kind == "muon":
            from mintext_b200.parallel.tp import current_tp

            tp = current_tp()
            tp_group = tp.group if (tp is not None and tp.size > 1) else None
        for n, p in params.items():
            g = grads.get(n)
            if g is None:
                continue
            g = g.float() * factor
            wd = cfg.weight_decay if weight_decay_mask(n) else 0.0
            view = muon_matrix_view(n, tuple(p.shape)) if self.kind == "muon" else None
            pf = p.float() if p.dtype != torch.float32 else p
            if view is None:
                oracle.adamw_update(pf, g, state.mu[n], state.nu[n], t, lr, cfg.adam_b1, cfg.adam_b2, cfg.adam_eps, wd)
            else:
                b, r, c = view
                beta = cfg.muon_beta
                mu = state.mu[n]
                mu.mul_(beta).add_(g, alpha=1 - beta)
                # Nesterov look-ahead with optax's bias correction of both terms
                mu_hat = (beta * mu / (1 - beta ** (t + 1))) + ((1 - beta) * g / (1 - beta ** t))
                axis = muon_slice_axis(n, p) if tp_group is not None else None
                if axis is not None:  # this rank holds a slice: the Gram matrices are summed over the group
                    upd, scale = muon_sliced_update(mu_hat, view, axis, tp_group, cfg.muon_newton_schulz_steps,
                                                    cfg.adam_eps, cfg.muon_consistent_rms)
                    upd = upd.reshape(p.shape)
                else:
                    upd = oracle.newton_schulz(mu_hat.reshape(b, r, c), cfg.muon_newton_schulz_steps,
                                               cfg.adam_eps).reshape(p.shape)
                    scale = muon_shape_scale(r, c, cfg.muon_consistent_rms)
                pf.add_(upd * scale + wd * pf, alpha=-lr)
            if pf is not p:
                p.copy_(pf)


def create_optimizer(config) -> Optimizer:
    return Optimizer(config)
