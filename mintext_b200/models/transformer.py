"""Decoder-only Transformer for every supported family (reference: mintext/models/base.py).

``DecoderLayer`` picks the attention flavour (Gated-Delta-Rule, MLA, or MHA/GQA with QK-norm / sliding window /
gating / local RoPE theta) and the feed-forward flavour (dense gated MLP, or MoE from layer
``first_k_dense_replace`` on when ``num_experts > 0``), with the 2-norm or Gemma 4-norm residual pattern.
``Transformer`` adds the embedding (optionally scaled by sqrt(D) in the compute dtype), the final norm and the
tied or untied output head with optional logit soft-capping.

Rematerialisation is a layer-granular checkpoint whose recompute pass can reuse named activations
(``query_proj``, ``key_proj``, ``value_proj``, ``out_proj``, ``mlp_gate_up``, ``mlp_down``) that the policy chose
to keep, optionally parked in pinned host memory in between.
"""

from __future__ import annotations

import torch
from torch import nn

from mintext_b200.modules.attention import Attention
from mintext_b200.modules.linear import MLP, Linear, normal_init
from mintext_b200.modules.linear_attention import GatedDeltaRuleAttention
from mintext_b200.modules.mla import MLAttention
from mintext_b200.modules.moe import MoEBlock
from mintext_b200.modules.norm import RMSNorm
from mintext_b200.ops import functional as F
from mintext_b200.utils.profiling import nvtx_range
from mintext_b200.ops.oracle import causal_mask

_QKV = frozenset({"query_proj", "key_proj", "value_proj"})
_ALL_DOTS = _QKV | {"out_proj", "mlp_gate_up", "mlp_down", "mlp_gate_proj", "mlp_up"}

# policy -> (names kept across the recompute, kept in pinned host memory?)
REMAT_POLICIES: dict[str, tuple[frozenset[str], bool] | None] = {
    "none": None,
    "full": (frozenset(), False),
    "minimal": (_ALL_DOTS, False),
    "save_qkv_proj": (_QKV, False),
    "save_dot_except_mlp": (_QKV | {"out_proj"}, False),
    "qkv_proj_offloaded": (_QKV, True),
    "minimal_offloaded": (_ALL_DOTS, True),
}


_BACKWARD_LAYER_HOOK = None


def set_backward_layer_hook(fn) -> None:
    """Install (or clear, with None) a callback ``fn(layer_index)`` that a forward pass arms on every decoder
    layer's input: it fires during the backward pass when the gradient of that input is complete, i.e. once every
    gradient kernel of the layer has been launched.  The training engine uses it on the last micro-batch of a step
    to start the layer's gradient reduce-scatter while the rest of the backward pass is still running."""
    global _BACKWARD_LAYER_HOOK
    _BACKWARD_LAYER_HOOK = fn


_FORWARD_LAYER_HOOK = None


def set_forward_layer_hook(fn) -> None:
    """Install (or clear, with None) a callback ``fn(layer_index)`` that every forward pass calls right before it
    enters a decoder layer.  The parameter-sharded engine mode uses it to make sure the layer's gathered weights
    have arrived and to start the gather of the next layer."""
    global _FORWARD_LAYER_HOOK
    _FORWARD_LAYER_HOOK = fn


def _arm_layer_hook(x: torch.Tensor, layer_index: int) -> None:
    if _FORWARD_LAYER_HOOK is not None:
        _FORWARD_LAYER_HOOK(layer_index)
    if _BACKWARD_LAYER_HOOK is None or not (torch.is_grad_enabled() and x.requires_grad):
        return

    def fire(grad, li=layer_index):
        hook = _BACKWARD_LAYER_HOOK
        if hook is not None:
            hook(li)
        return None

    x.register_hook(fire)


def make_causal_mask(seq_len: int, dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """Additive ``[1,1,S,S]`` causal mask (0 / -1e10)."""
    return causal_mask(seq_len, dtype)


def _all_layers_scannable(config) -> bool:
    """True when every layer has the same structure and none is MoE: the condition under which the reference
    stacks layer parameters along a leading axis.  Kept because it decides the checkpoint tree layout the
    HF converter has to understand; execution here is always an ordinary loop."""
    if not config.scan_layers or config.num_experts > 0:
        return False
    return len(set(config.layer_types)) <= 1


class _LayerCheckpoint(torch.autograd.Function):
    """Run a layer without recording its graph; re-run it in backward.  Named activations selected by the
    policy survive in a RematContext so the recompute skips the GEMMs that produced them."""

    @staticmethod
    def forward(ctx, run_fn, rctx, x, *params):
        ctx.run_fn = run_fn
        ctx.rctx = rctx
        ctx.save_for_backward(x)
        ctx.cpu_rng = torch.get_rng_state()
        with torch.no_grad(), F.remat_scope(rctx):
            out = run_fn(x)
        return out

    @staticmethod
    def backward(ctx, *grads):
        (x,) = ctx.saved_tensors
        xd = x.detach().requires_grad_(x.requires_grad)
        ctx.rctx.start_replay()
        with torch.enable_grad(), F.remat_scope(ctx.rctx):
            out = ctx.run_fn(xd)
        outs = out if isinstance(out, tuple) else (out,)
        pairs = [(o, g) for o, g in zip(outs, grads) if isinstance(o, torch.Tensor) and o.requires_grad and g is not None]
        params = [p for p in ctx.run_fn.params if p.requires_grad]
        inputs = ([xd] if xd.requires_grad else []) + params
        got = torch.autograd.grad([o for o, _ in pairs], inputs, [g for _, g in pairs], allow_unused=True)
        got = list(got)
        dx = got.pop(0) if xd.requires_grad else None
        by_param = dict(zip(params, got))
        ctx.rctx.store.clear()
        return (None, None, dx) + tuple(by_param.get(p) for p in ctx.run_fn.params)


class _LayerRunner:
    def __init__(self, layer, positions, mask, default_positions):
        self.layer, self.positions, self.mask, self.default_positions = layer, positions, mask, default_positions
        self.params = list(layer.parameters())
        self.aux = None

    def __call__(self, x):
        y, aux = self.layer(x, self.positions, self.mask, self.default_positions)
        if aux is not None and self.aux is None:
            self.aux = {k: v.detach() if isinstance(v, torch.Tensor) and k != "aux_loss" else v for k, v in aux.items()}
        return y


def apply_layer_with_remat(layer, x, positions, mask, policy: str, default_positions: bool = False):
    spec = REMAT_POLICIES[policy]
    if spec is None or not torch.is_grad_enabled():
        return layer(x, positions, mask, default_positions)
    runner = _LayerRunner(layer, positions, mask, default_positions)
    rctx = F.RematContext(spec[0], offload=spec[1])
    y = _LayerCheckpoint.apply(runner, rctx, x, *runner.params)
    return y, runner.aux


class DecoderLayer(nn.Module):
    def __init__(self, config, layer_idx: int, *, rngs=None, mesh=None):
        super().__init__()
        dt = config.torch_dtype
        layer_type = config.layer_types[layer_idx] if config.layer_types else "full_attention"
        self.use_post_ffw_norm = config.use_post_ffw_norm
        D, eps = config.hidden_size, config.rms_norm_eps
        self.pre_attn_norm = RMSNorm(D, eps, dt)
        self.post_attn_norm = RMSNorm(D, eps, dt)
        if self.use_post_ffw_norm:
            self.pre_ffw_norm = RMSNorm(D, eps, dt)
            self.post_ffw_norm = RMSNorm(D, eps, dt)
        self.is_linear = layer_type == "linear_attention"
        self.has_moe = config.num_experts > 0 and layer_idx >= config.first_k_dense_replace
        # Under tensor parallelism the residual stream is sharded over tokens.  Dense attention, multi-head-latent
        # attention and the Gated Delta Rule shard their heads, dense MLPs (and a mixture-of-experts block's shared
        # expert) their hidden columns; the router and the routed experts simply work on the rank's own token shard
        # (the group acts as data parallelism for them).  A sub-layer without any of these paths could still be
        # computed in full on every rank of the group (parallel/tp.py::run_replicated); none is at present.
        self.attn_replicated = False
        self.mlp_replicated = False
        if self.is_linear:
            self.attention = GatedDeltaRuleAttention(config, rngs=rngs)
        elif config.attention_type == "mla":
            self.attention = MLAttention(config, layer_idx, rngs=rngs)
        else:
            sliding = config.sliding_window if layer_type == "sliding_attention" else None
            local_theta = config.rope_local_theta if (sliding is not None and config.model_type == "gemma3") else None
            self.attention = Attention(
                config, rngs=rngs, mesh=mesh, use_qk_norm=config.use_qk_norm, sliding_window=sliding,
                use_gate=(config.model_type == "qwen3_next" and layer_type == "full_attention"),
                rope_local_theta=local_theta)
        self.mlp = MoEBlock(config, rngs=rngs) if self.has_moe else MLP(config, rngs=rngs, mesh=mesh)

    def _attend(self, h, positions, mask, default_positions):
        if self.attn_replicated:
            from mintext_b200.parallel import tp as tpm

            fn = self.attention if self.is_linear else (lambda t: self.attention(t, positions, mask, default_positions))
            return tpm.run_replicated(fn, h, tpm.current_tp())[0]
        if self.is_linear:
            return self.attention(h)
        return self.attention(h, positions, mask, default_positions)

    def _ffw(self, h):
        if self.mlp_replicated:
            from mintext_b200.parallel import tp as tpm

            return tpm.run_replicated(self.mlp, h, tpm.current_tp())
        if self.has_moe:
            return self.mlp(h)
        return self.mlp(h), None

    def forward(self, x, positions=None, mask=None, default_positions: bool = False, pending=None,
                defer_residual: bool = False):
        """``pending`` is a feed-forward output of the previous layer that has not been added to ``x`` yet: it is
        folded into this layer's first norm (one pass over memory instead of a separate add).  With
        ``defer_residual`` the layer likewise returns ``(x, aux, own pending output)`` instead of adding it."""
        if self.use_post_ffw_norm:
            if pending is not None:
                x = x + pending
            h = self.post_attn_norm(self._attend(self.pre_attn_norm(x), positions, mask, default_positions))
            x = x + h
            h, aux = self._ffw(self.pre_ffw_norm(x))
            x = x + self.post_ffw_norm(h)
            return (x, aux, None) if defer_residual else (x, aux)
        if pending is not None:
            n, x = self.pre_attn_norm.forward_add(pending, x)
        else:
            n = self.pre_attn_norm(x)
        a = self._attend(n, positions, mask, default_positions)
        h, x = self.post_attn_norm.forward_add(a, x)  # x <- x + a ; h <- norm(x), one pass
        h, aux = self._ffw(h)
        if defer_residual:
            return x, aux, h
        return x + h, aux


class Transformer(nn.Module):
    """``forward(tokens, positions, mask=None, return_hidden=False) -> (logits | hidden, aux_list)``."""

    def __init__(self, config, *, rngs: torch.Generator | int | None = None, mesh=None):
        super().__init__()
        if isinstance(rngs, int) or rngs is None:
            gen = torch.Generator(device="cpu")
            gen.manual_seed(int(rngs) if rngs is not None else int(config.seed))
            rngs = gen
        self.config = config
        self.final_logit_softcapping = config.final_logit_softcapping
        dt, wdt = config.torch_dtype, config.torch_weight_dtype
        self.embedding_scale = float(config.hidden_size) ** 0.5 if config.scale_embeddings else None
        V, D = config.vocab_size, config.hidden_size
        self.token_embedder = nn.Parameter(normal_init((V, D), 0.02, rngs, wdt))
        self.token_embedder.logical_axes = ("vocab", "embed")
        self.layers = nn.ModuleList(
            [DecoderLayer(config, i, rngs=rngs, mesh=mesh) for i in range(config.num_hidden_layers)])
        self.has_tp_replicated = any(l.attn_replicated or l.mlp_replicated for l in self.layers)
        self.remat_policy = config.remat_policy
        self.final_norm = RMSNorm(D, config.rms_norm_eps, dt)
        self.tie_word_embeddings = config.tie_word_embeddings
        if not config.tie_word_embeddings:
            self.output_proj = Linear(D, V, dt, wdt, ("embed", "vocab"), rngs=rngs)
        self._use_scan = _all_layers_scannable(config)
        # vocabulary-parallel ends (parallel/vocab_parallel.py): this rank keeps rows [v_lo, v_hi) of the embedding
        # table and the same columns of the output projection
        from mintext_b200.parallel.tp import current_tp

        tp = current_tp()
        self.vocab_parallel = bool(getattr(config, "tp_vocab_parallel", False)) and tp is not None and tp.size > 1
        if self.vocab_parallel:
            from mintext_b200.parallel.vocab_parallel import shard_vocab_rows

            owners = [(self, "token_embedder", 0)]
            if not config.tie_word_embeddings:
                owners.append((self.output_proj, "kernel", 1))
            for owner, attr, dim in owners:
                full = getattr(owner, attr)
                local = nn.Parameter(shard_vocab_rows(full.data, tp, dim))
                local.logical_axes = full.logical_axes
                local.tensor_parallel = True
                local.shard_spec = (dim, tp.rank, tp.size)
                setattr(owner, attr, local)

    # the output head as (weight, weight_is_[vocab, hidden]) for the fused projection + loss path
    def output_weight(self) -> tuple[torch.Tensor, bool]:
        if self.tie_word_embeddings:
            return self.token_embedder, True
        return self.output_proj.kernel, False

    def forward(self, tokens: torch.Tensor, positions: torch.Tensor | None = None, mask: torch.Tensor | None = None,
                return_hidden: bool = False, default_positions: bool | None = None):
        cfg = self.config
        dt = cfg.torch_dtype
        if default_positions is None:
            default_positions = positions is None
        if positions is None:
            positions = torch.arange(tokens.shape[1], device=tokens.device)[None].expand(tokens.shape[0], -1)
        from mintext_b200.parallel.tp import current_tp

        tp = current_tp()
        if tp is not None and tp.size > 1:
            # token-sharded residual stream: this rank embeds (and later scores) rows [lo, hi) of the flat tokens
            B, S = tokens.shape
            tp.batch_shape = (B, S)
            lo, hi = tp.shard(B * S, "tokens per batch")
            tokens = tokens.reshape(1, B * S)[:, lo:hi]
        if self.vocab_parallel:
            from mintext_b200.parallel import vocab_parallel as vp

            x = vp.embedding(self.token_embedder, tokens, tp, dt, self.embedding_scale)
        else:
            x = F.embedding(self.token_embedder, tokens, dt, self.embedding_scale)
        all_aux = []
        pending = None
        fuse = REMAT_POLICIES[self.remat_policy] is None or not torch.is_grad_enabled()
        for li, layer in enumerate(self.layers):
            _arm_layer_hook(x, li)
            with nvtx_range(f"layer{li}"):
                if fuse:  # carry the last residual add into the next norm kernel
                    x, aux, pending = layer(x, positions, mask, default_positions, pending=pending, defer_residual=True)
                else:
                    x, aux = apply_layer_with_remat(layer, x, positions, mask, self.remat_policy, default_positions)
            all_aux.append(aux)
        if pending is not None:
            x, _ = self.final_norm.forward_add(pending, x)
        else:
            x = self.final_norm(x)
        if return_hidden:
            return x, all_aux
        if self.vocab_parallel:
            raise NotImplementedError("with tp_vocab_parallel no rank holds the whole output head: ask for the hidden "
                                      "states (return_hidden=True) and score them with "
                                      "parallel.vocab_parallel.linear_cross_entropy, as trainer.compute_loss does")
        if self.tie_word_embeddings:
            logits = F.linear_nt(x, self.token_embedder, dtype=dt)
        else:
            logits = self.output_proj(x)
        if self.final_logit_softcapping is not None:
            cap = self.final_logit_softcapping
            logits = torch.tanh(logits / cap) * cap
        return logits, all_aux
