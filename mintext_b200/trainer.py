"""Loss functions, train / eval steps and the train state (reference: mintext/trainer.py).

This module is the device-agnostic statement of a training step: it works on any model built from
:mod:`mintext_b200.models` with ordinary autograd and the per-tensor optimizer, which is what the CPU plumbing
config and the unit tests run.  On B200 the same loss code runs under :class:`mintext_b200.parallel.engine.
TrainEngine`, which replaces the optimizer step with the fused, sharded kernels.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch

from mintext_b200.models.transformer import make_causal_mask
from mintext_b200.ops import functional as F
from mintext_b200.ops import oracle
from mintext_b200.optim import accumulate_gradients, create_lr_schedule, create_optimizer


@dataclass
class TrainState:
    """``step`` counts optimizer updates; ``params`` is the model's ``{dotted name: Parameter}`` dict (the same
    tensors the model computes with); ``opt_state`` and ``tx`` belong to the optimizer."""

    step: int
    params: dict[str, torch.Tensor]
    opt_state: Any
    tx: Any

    params_only_restore: bool = False
    # process groups of a multi-process run (None: single process, or every rank trains on its own)
    groups: "ReduceGroups | None" = None

    # ---- checkpoint protocol (see mintext_b200.checkpoint.manager)
    def _slice_entry(self, name: str, tensor: torch.Tensor):
        """A parameter of which this rank holds a slice is saved as one shard per slice (same entry format as the GPU
        engine's), written by the first of the ranks that hold the slice; whole tensors by rank 0."""
        p = self.params[name]
        spec = getattr(p, "shard_spec", None)
        if spec is None or not _is_slice(p):
            return tensor
        import torch.distributed as dist

        grp = self.groups.replica_group(p) if self.groups is not None else None
        first = grp is None or dist.get_rank(grp) == 0
        me = dist.get_rank() if dist.is_available() and dist.is_initialized() else 0
        dim, idx, cnt = (int(v) for v in spec)
        return {"tensor": tensor, "writer_rank": me if first else -1, "shard": (dim, idx, cnt),
                "suffix": f".shard{idx}of{cnt}"}

    def _shard_of(self, name: str):
        p = self.params[name]
        spec = getattr(p, "shard_spec", None)
        return tuple(int(v) for v in spec) if (spec is not None and _is_slice(p)) else None

    def checkpoint_tree(self) -> dict:
        tree: dict = {"step": self.step, "opt_state/count": self.opt_state.count}
        for n, p in self.params.items():
            tree[f"params/{n}"] = self._slice_entry(n, p.detach())
        for n, t in self.opt_state.mu.items():
            tree[f"opt_state/mu/{n}"] = self._slice_entry(n, t)
        for n, t in self.opt_state.nu.items():
            tree[f"opt_state/nu/{n}"] = self._slice_entry(n, t)
        return tree

    @torch.no_grad()
    def load_checkpoint_tree(self, read) -> None:
        def get(path, name):
            spec = self._shard_of(name)
            return read(path, shard=spec) if spec is not None else read(path)

        for n, p in self.params.items():
            p.copy_(get(f"params/{n}", n).to(p.dtype))
        if self.params_only_restore:
            return
        self.step = int(read("step"))
        self.opt_state.count = int(read("opt_state/count"))
        for n in self.opt_state.mu:
            self.opt_state.mu[n].copy_(get(f"opt_state/mu/{n}", n))
        for n in self.opt_state.nu:
            self.opt_state.nu[n].copy_(get(f"opt_state/nu/{n}", n))

    def reset_step(self) -> None:
        self.step = 0
        self.opt_state = self.tx.init({n: p for n, p in self.params.items() if p.requires_grad})

    def refresh_from_model(self) -> None:
        """Parameters are shared with the model, nothing to copy."""


# ------------------------------------------------------------------------------------------ multi-process runs
@dataclass
class ReduceGroups:
    """Who averages what in a multi-process run of this trainer (the CPU statement of what the GPU engine does).

    Every rank's loss is the mean over its own tokens, so the job's loss is the mean over ranks.  A replicated
    parameter's gradient is therefore the sum over all ranks divided by the rank count.  A parameter of which a rank
    holds a slice (tensor-, vocabulary- or expert-parallel) already receives, through the backward pass of the
    collectives, the contributions of every rank that used the slice; what is left is the sum over the ranks that hold
    *the same* slice (``slice_group``; ``expert_group`` for expert slices when tensor and expert parallelism are
    combined; None: the slice is unique) and the same division by the rank count."""

    world: Any = None          # all ranks (None: the default group)
    slice_group: Any = None
    expert_group: Any = None

    def replica_group(self, p):
        if getattr(p, "expert_parallel", False) and self.expert_group is not None:
            return self.expert_group
        return self.slice_group


def _is_slice(p) -> bool:
    return bool(getattr(p, "tensor_parallel", False) or getattr(p, "expert_parallel", False))


def _group_size(group) -> int:
    import torch.distributed as dist

    return dist.get_world_size(group) if group is not None else 1


@torch.no_grad()
def sync_gradients(grads: dict, params: dict, groups: ReduceGroups) -> dict:
    """Average ``grads`` over the job as :class:`ReduceGroups` describes (missing gradients count as zeros, so every
    rank takes part in every collective).  Returns the new dict."""
    import torch.distributed as dist

    world = dist.get_world_size(groups.world)
    out = {n: (g if g is not None else torch.zeros_like(params[n])) for n, g in grads.items()}
    by_group: dict[int, tuple] = {}
    for n, g in out.items():
        p = params[n]
        grp = groups.replica_group(p) if _is_slice(p) else groups.world
        if _is_slice(p) and grp is None:
            continue  # a slice nobody else holds
        by_group.setdefault(id(grp), (grp, []))[1].append(n)
    for grp, names in by_group.values():  # one collective per group, over a flat copy
        flat = torch.cat([out[n].reshape(-1).float() for n in names])
        dist.all_reduce(flat, group=grp)
        off = 0
        for n in names:
            k = out[n].numel()
            out[n] = flat[off:off + k].view(out[n].shape).to(out[n].dtype)
            off += k
    return {n: g / world for n, g in out.items()}


@torch.no_grad()
def global_l2_norm(tensors: dict, params: dict, groups: ReduceGroups) -> torch.Tensor:
    """L2 norm of a job-wide tree of which ranks hold replicas and slices: replicated tensors count once, every
    distinct slice once."""
    import torch.distributed as dist

    rep = torch.zeros((), dtype=torch.float32)
    sl = torch.zeros((), dtype=torch.float32)
    for n, t in tensors.items():
        if t is None:
            continue
        s = (t.detach().float() ** 2).sum()
        if _is_slice(params[n]):
            sl += s / _group_size(groups.replica_group(params[n]))
        else:
            rep += s
    dist.all_reduce(sl, group=groups.world)
    return torch.sqrt(rep + sl)


# ------------------------------------------------------------------------------------------ losses
def cross_entropy_with_z_loss(logits: torch.Tensor, targets: torch.Tensor, label_smoothing: float = 0.0,
                              z_loss_weight: float = 0.0):
    """Per-token ``(loss incl. z-loss, z-loss)`` from fp32 log-softmax."""
    return oracle.cross_entropy(logits, targets, label_smoothing, z_loss_weight)


def cross_entropy_loss(logits: torch.Tensor, targets: torch.Tensor, label_smoothing: float = 0.0,
                       z_loss_weight: float = 0.0):
    """logits ``[B,S,V]``, targets ``[B,S]`` -> ``(loss [B,S], z_loss [B,S])``."""
    return oracle.cross_entropy(logits, targets, label_smoothing, z_loss_weight)


def chunked_cross_entropy_loss(hidden_states: torch.Tensor, targets: torch.Tensor, output_proj, num_tiles: int,
                               label_smoothing: float = 0.0, z_loss_weight: float = 0.0):
    """Project-and-score ``num_tiles`` token chunks one at a time so the full ``[N,V]`` logits never exist.
    ``output_proj`` maps ``[n,D] -> [n,V]``."""
    hidden = hidden_states
    N = hidden.shape[0]
    step = N // num_tiles
    losses, zs = [], []
    for i in range(num_tiles):
        sl = slice(i * step, (i + 1) * step if i < num_tiles - 1 else N)
        l, z = oracle.cross_entropy(output_proj(hidden[sl]), targets[sl], label_smoothing, z_loss_weight)
        losses.append(l)
        zs.append(z)
    return torch.cat(losses), torch.cat(zs)


def _l2_norm(tensors) -> torch.Tensor:
    ts = [t for t in tensors if t is not None]
    return torch.sqrt(sum((t.detach().float() ** 2).sum() for t in ts))


# ------------------------------------------------------------------------------------------ loss
def compute_loss(params, model, config, batch, loss_scale: float | None = None):
    """Forward + loss on one batch ``{"input_tokens", "target_tokens"}`` ``[B,S]``.

    Returns ``(loss, aux)`` with ``aux = {loss, z_loss, per_token_loss, moe_expert_counts}``.  The loss is the
    mean over all ``B*S`` tokens (no padding mask).  ``params`` is accepted for signature parity; the model
    already computes with those tensors.
    """
    tokens, targets = batch["input_tokens"], batch["target_tokens"]
    B, S = tokens.shape
    mask = None
    if config.attn_logit_softcapping is not None and not tokens.is_cuda:
        mask = make_causal_mask(S).to(tokens.device)
    fused = F.use_cuda(model.final_norm.scale.new_empty(0, dtype=config.torch_dtype)) and tokens.is_cuda
    from mintext_b200.parallel.tp import current_tp

    tp = current_tp()
    vocab_parallel = bool(getattr(model, "vocab_parallel", False))
    hidden_mode = fused or config.num_vocab_tiles > 1 or vocab_parallel
    out, aux_list = model(tokens, None, mask, return_hidden=hidden_mode)
    if tp is not None and tp.size > 1:  # the model returned this rank's token shard
        lo, hi = tp.shard(B * S, "tokens per batch")
        targets = targets.reshape(1, B * S)[:, lo:hi]
        B, S = 1, hi - lo
    ntok = B * S
    scale = loss_scale if loss_scale is not None else 1.0 / ntok
    if vocab_parallel:  # the head is sharded over the vocabulary: softmax statistics are reduced over the group
        from mintext_b200.parallel.vocab_parallel import linear_cross_entropy as vp_linear_cross_entropy

        w, is_vd = model.output_weight()
        per_tok, z = vp_linear_cross_entropy(
            out.reshape(ntok, -1), w, targets.reshape(-1), tp, is_vd, config.label_smoothing, config.z_loss_weight,
            config.final_logit_softcapping, chunks=max(int(config.num_vocab_tiles), 1))
        per_tok, z = per_tok.view(B, S), z.view(B, S)
        loss = per_tok.sum() * scale
    elif fused:
        w, is_vd = model.output_weight()
        per_tok, z = F.linear_cross_entropy(
            out.reshape(ntok, -1), w, targets.reshape(-1), weight_is_vd=is_vd,
            label_smoothing=config.label_smoothing, z_loss_weight=config.z_loss_weight,
            softcap=config.final_logit_softcapping, loss_scale=scale)
        per_tok, z = per_tok.view(B, S), z.view(B, S)
        loss = per_tok.sum() * scale
    elif config.num_vocab_tiles > 1:
        w, is_vd = model.output_weight()
        cap = config.final_logit_softcapping

        def proj(h):
            lg = F.linear_nt(h, w, dtype=config.torch_dtype) if is_vd else F.linear(h, w, dtype=config.torch_dtype)
            return torch.tanh(lg / cap) * cap if cap is not None else lg

        per_tok, z = chunked_cross_entropy_loss(out.reshape(ntok, -1), targets.reshape(-1), proj,
                                                config.num_vocab_tiles, config.label_smoothing,
                                                config.z_loss_weight)
        per_tok, z = per_tok.view(B, S), z.view(B, S)
        loss = per_tok.mean()
    else:
        per_tok, z = cross_entropy_loss(out, targets, config.label_smoothing, config.z_loss_weight)
        loss = per_tok.mean()
    counts = []
    aux_loss = None
    for aux in aux_list:
        if aux is None:
            continue
        counts.append(oracle.histogram(aux["topk_indices"], config.num_experts))
        if "aux_loss" in aux and config.router_aux_loss_coef > 0:
            aux_loss = aux["aux_loss"] if aux_loss is None else aux_loss + aux["aux_loss"]
    if aux_loss is not None:
        # Sub-layers that a tensor-parallel group computes in full on every rank (parallel/tp.py::run_replicated;
        # none at present) form the auxiliary loss of the whole batch on every rank while the token loss is the rank's
        # share; the engine averages the ranks' gradients, so such a replicated term counts group-size times here.
        # Token-sharded routers contribute their own share, like the token loss.
        rep = 1.0
        if getattr(model, "has_tp_replicated", False):
            from mintext_b200.parallel.tp import current_tp

            tp = current_tp()
            rep = float(tp.size) if (tp is not None and tp.size > 1) else 1.0
        term = config.router_aux_loss_coef * aux_loss * (scale * ntok)
        reported = (loss + term).detach()          # what a single process would report
        loss = loss + term * rep
    else:
        reported = loss.detach()
    out_aux = {
        "loss": reported,
        "z_loss": z.detach().mean(),
        "per_token_loss": per_tok.detach(),
        "moe_expert_counts": torch.stack(counts) if counts else None,
    }
    return loss, out_aux


# ------------------------------------------------------------------------------------------ steps
def create_train_state(model, config, groups: ReduceGroups | None = None) -> TrainState:
    params = dict(model.named_parameters())
    tx = create_optimizer(config)
    trainable = {n: p for n, p in params.items() if p.requires_grad}
    return TrainState(step=0, params=params, opt_state=tx.init(trainable), tx=tx, groups=groups)


def _active_groups(state) -> ReduceGroups | None:
    groups = getattr(state, "groups", None)
    if groups is None:
        return None
    import torch.distributed as dist

    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(groups.world) < 2:
        return None
    return groups


def train_step(state: TrainState, batch, model, config):
    """One optimizer update.  Metrics: ``loss``, ``z_loss``, ``learning_rate`` (schedule value at the
    pre-update step), ``grad_norm`` (before clipping), ``param_norm`` (before the update), ``moe_expert_counts``."""
    trainable = {n: p for n, p in state.params.items() if p.requires_grad}
    n_acc = int(config.gradient_accumulation_steps)
    if n_acc > 1:
        loss, aux, grads = accumulate_gradients(
            lambda _p, mb: compute_loss(_p, model, config, mb), trainable, batch, n_acc)
    else:
        loss, aux = compute_loss(state.params, model, config, batch)
        got = torch.autograd.grad(loss, list(trainable.values()), allow_unused=True)
        grads = dict(zip(trainable, got))
        loss = loss.detach()
    groups = _active_groups(state)
    if groups is not None:
        import torch.distributed as dist

        grads = sync_gradients(grads, trainable, groups)
        grad_norm = global_l2_norm(grads, trainable, groups)
        param_norm = global_l2_norm(state.params, state.params, groups)
        loss = loss.clone()
        dist.all_reduce(loss, group=groups.world)
        loss /= dist.get_world_size(groups.world)
        zl = aux["z_loss"].clone()
        dist.all_reduce(zl, group=groups.world)
        aux["z_loss"] = zl / dist.get_world_size(groups.world)
        if aux.get("moe_expert_counts") is not None:  # the load-balancing update looks at the whole job's tokens
            counts = aux["moe_expert_counts"].clone()
            dist.all_reduce(counts, group=groups.world)
            aux["moe_expert_counts"] = counts
    else:
        grad_norm = _l2_norm(grads.values())
        param_norm = _l2_norm(state.params.values())
    lr = create_lr_schedule(config)(state.step)
    skipped = False
    if getattr(config, "nan_policy", "ignore") != "ignore":
        from mintext_b200.parallel.health import apply_nan_policy

        skipped = apply_nan_policy(config.nan_policy, float(loss), state.step)
    if not skipped:
        state.tx.update(trainable, grads, state.opt_state, state.step,
                        grad_norm=float(grad_norm) if groups is not None else None)
        state.step += 1
    metrics = {
        "skipped": skipped,
        "loss": loss,
        "z_loss": aux["z_loss"],
        "learning_rate": lr,
        "grad_norm": grad_norm,
        "param_norm": param_norm,
        "moe_expert_counts": aux.get("moe_expert_counts"),
    }
    return state, metrics


@torch.no_grad()
def eval_step(state: TrainState, batch, model, config) -> dict:
    loss, _ = compute_loss(state.params, model, config, batch)
    return {"eval_loss": loss.detach()}


@torch.no_grad()
def update_expert_biases(state: TrainState, expert_counts: torch.Tensor | None, config) -> TrainState:
    """Loss-free balancing: per MoE layer (in layer order) ``bias += rate * sign(mean_count - count)``."""
    if expert_counts is None:
        return state
    rate = config.e_score_correction_bias_update_rate
    names = sorted((n for n in state.params if n.endswith("e_score_correction_bias")),
                   key=lambda n: int(n.split(".")[1]))
    for name, counts in zip(names, expert_counts):
        c = counts.float()
        state.params[name].add_(rate * torch.sign(c.mean() - c).to(state.params[name].device))
    return state
