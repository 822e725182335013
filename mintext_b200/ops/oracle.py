"""Plain-PyTorch statement of every op's math.

These functions are (a) the numerical oracle each CUDA kernel is tested against, (b) the execution path on
machines without a GPU (the CPU plumbing config runs on them), and (c) differentiable through autograd, so
they also serve as the backward oracle.  The dtype contracts follow the reference modules file by file; the
docstring of each function names the reference site it restates.
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F


# ----------------------------------------------------------------------------- norm
def rms_norm(x: torch.Tensor, scale: torch.Tensor, eps: float, dtype: torch.dtype | None = None) -> torch.Tensor:
    """fp32 statistics; the normalised value is cast to ``dtype`` first and then multiplied by the cast scale
    (mintext/modules/norm.py:21-25)."""
    dtype = dtype or x.dtype
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return y.to(dtype) * scale.to(dtype)


# ----------------------------------------------------------------------------- activations
def activation(name: str):
    """silu / gelu (erf) / gelu_pytorch_tanh / relu (mintext/modules/linear.py:153-158)."""
    table = {
        "silu": F.silu,
        "gelu": F.gelu,
        "gelu_pytorch_tanh": lambda t: F.gelu(t, approximate="tanh"),
        "relu": F.relu,
    }
    if name not in table:
        raise ValueError(f"Unknown activation: {name}")
    return table[name]


def histogram(indices: torch.Tensor, bins: int) -> torch.Tensor:
    """Occurrences of ``0..bins-1`` in ``indices`` (int64).  Unlike ``torch.bincount`` this never copies a size back
    to the host, so the launching thread keeps running ahead of the device."""
    flat = indices.reshape(-1)
    return torch.zeros(bins, dtype=torch.int64, device=flat.device).scatter_add_(0, flat, torch.ones_like(flat))


ACT_CODES = {"silu": 0, "gelu_pytorch_tanh": 1, "gelu": 2, "relu": 3}


def gated_act(gate_up: torch.Tensor, act: str) -> torch.Tensor:
    g, u = gate_up.chunk(2, dim=-1)
    return activation(act)(g) * u


# ----------------------------------------------------------------------------- rope
def _yarn_correction_dim(rot: float, dim: int, base: float, max_pos: int) -> float:
    return dim * math.log(max_pos / (rot * 2 * math.pi)) / (2 * math.log(base))


def compute_inv_freq(config, dim: int, theta: float | None = None) -> tuple[torch.Tensor, float]:
    """Inverse frequencies ``[dim/2]`` and the attention factor for default / linear / yarn / llama3 scaling
    (mintext/modules/rope.py:53-142)."""
    base = float(theta if theta is not None else config.rope_theta)
    orig = config.rope_original_max_position_embeddings or config.seq_length
    exponents = torch.arange(0, dim, 2, dtype=torch.float32) / dim
    pos_freqs = base ** exponents
    kind = config.rope_type
    factor = float(config.rope_scaling_factor)
    if kind == "default":
        return 1.0 / pos_freqs, 1.0
    if kind == "linear":
        return 1.0 / (factor * pos_freqs), 1.0
    if kind == "yarn":
        low = max(math.floor(_yarn_correction_dim(config.rope_yarn_beta_fast, dim, base, orig)), 0)
        high = min(math.ceil(_yarn_correction_dim(config.rope_yarn_beta_slow, dim, base, orig)), dim - 1)
        hi = high + 0.001 if low == high else high
        ramp = ((torch.arange(dim // 2, dtype=torch.float32) - low) / (hi - low)).clamp(0.0, 1.0)
        keep = 1.0 - ramp
        inv = (1.0 / (factor * pos_freqs)) * (1 - keep) + (1.0 / pos_freqs) * keep
        if factor <= 1.0:
            att = 1.0
        elif config.rope_yarn_mscale_all_dim > 0:
            att = (0.1 * config.rope_yarn_mscale * math.log(factor) + 1.0) / (
                0.1 * config.rope_yarn_mscale_all_dim * math.log(factor) + 1.0
            )
        else:
            att = 0.1 * math.log(factor) + 1.0
        return inv, att
    if kind == "llama3":
        inv = 1.0 / pos_freqs
        wavelen = 2 * math.pi / inv
        lo_f, hi_f = config.rope_llama3_low_freq_factor, config.rope_llama3_high_freq_factor
        low_wl, high_wl = orig / lo_f, orig / hi_f
        scaled = torch.where(wavelen > low_wl, inv / factor, inv)
        smooth = (orig / wavelen - lo_f) / (hi_f - lo_f)
        blended = (1 - smooth) * scaled / factor + smooth * scaled
        medium = ~(wavelen < high_wl) & ~(wavelen > low_wl)
        return torch.where(medium, blended, scaled), 1.0
    raise ValueError(f"Unknown rope_type: {kind}")


def rope_tables(inv_freq: torch.Tensor, attention_factor: float, max_pos: int, device=None) -> tuple[torch.Tensor, torch.Tensor]:
    """cos / sin tables ``[max_pos, rot/2]`` in fp32, attention factor folded in."""
    pos = torch.arange(max_pos, dtype=torch.float32, device=device)
    ang = pos[:, None] * inv_freq.to(device)[None, :]
    return (ang.cos() * attention_factor).contiguous(), (ang.sin() * attention_factor).contiguous()


def apply_rope(x: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor, attention_factor: float,
               rot_dim: int, interleave: bool) -> torch.Tensor:
    """x ``[B,S,H,d]``, positions ``[B,S]``.  fp32 math, duplicated ``[sin,sin]`` / ``[cos,cos]`` tables, untouched
    tail when ``rot_dim < d``, result cast back to x.dtype (mintext/modules/rope.py:190-232).  ``interleave``
    follows the HuggingFace DeepSeek-V3 definition (de-interleave, then half rotation) rather than the
    reference's pair-swap with duplicated tables, which does not rotate pairs by a common angle."""
    full = x.shape[-1]
    xr = x[..., :rot_dim]
    ang = positions[:, :, None, None].float() * inv_freq.to(x.device)
    sin = torch.cat([ang.sin(), ang.sin()], -1) * attention_factor
    cos = torch.cat([ang.cos(), ang.cos()], -1) * attention_factor
    xf = xr.float()
    if interleave:
        # pairs (2i, 2i+1) are brought to the half layout (evens first, then odds) and rotated there; q and k get
        # the same permutation, so attention scores equal those of an interleaved rotation (HF DeepSeek-V3)
        xf = xf.reshape(*xf.shape[:-1], -1, 2).transpose(-1, -2).reshape(xf.shape)
    half = rot_dim // 2
    rot = torch.cat([-xf[..., half:], xf[..., :half]], dim=-1)
    out = xf * cos + rot * sin
    if rot_dim < full:
        out = torch.cat([out, x[..., rot_dim:].float()], dim=-1)
    return out.to(x.dtype)


# ----------------------------------------------------------------------------- attention
NEG_INF = -1e10


def causal_mask(seq_len: int, dtype=torch.float32, device=None) -> torch.Tensor:
    """Additive ``[1,1,S,S]`` mask, 0 where attending is allowed and -1e10 elsewhere (mintext/models/base.py:331-339)."""
    allowed = torch.tril(torch.ones(seq_len, seq_len, dtype=torch.bool, device=device))
    return torch.where(allowed, 0.0, NEG_INF).to(dtype)[None, None]


def sliding_window_mask(seq_len: int, window: int, dtype=torch.float32, device=None) -> torch.Tensor:
    """Additive mask keeping ``0 <= i - j < window`` (mintext/modules/attention.py:94-100; HF semantics)."""
    i = torch.arange(seq_len, device=device)[:, None]
    j = torch.arange(seq_len, device=device)[None, :]
    allowed = (i - j >= 0) & (i - j < window)
    return torch.where(allowed, 0.0, NEG_INF).to(dtype)[None, None]


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, causal: bool = True,
              window: int | None = None, softcap: float | None = None, mask: torch.Tensor | None = None) -> torch.Tensor:
    """q ``[B,S,H,d]``, k/v ``[B,S,Hkv,d(v)]`` -> ``[B,S,H,dv]``.  Grouped-query heads share K/V without
    repeating them; scores and softmax in fp32, probabilities cast to the input dtype before ``P @ V``
    (mintext/modules/attention.py:304-358, mintext/modules/mla.py:129-143)."""
    B, S, H, d = q.shape
    Hkv = k.shape[2]
    G = H // Hkv
    qg = q.permute(0, 2, 1, 3).reshape(B, Hkv, G, S, d)
    kt = k.permute(0, 2, 1, 3)
    vt = v.permute(0, 2, 1, 3)
    scores = torch.einsum("bngsd,bntd->bngst", qg, kt) * scale
    scores = scores.float()
    if softcap is not None:
        scores = torch.tanh(scores / softcap) * softcap
    Sk = k.shape[1]
    if causal:
        scores = scores + causal_mask(Sk, device=q.device)[:, :, None][..., -S:, :]
    if window is not None:
        scores = scores + sliding_window_mask(Sk, window, device=q.device)[:, :, None][..., -S:, :]
    if mask is not None:
        scores = scores + mask[:, :, None].float()
    probs = torch.softmax(scores, dim=-1).to(q.dtype)
    out = torch.einsum("bngst,bntd->bngsd", probs, vt)
    return out.reshape(B, H, S, v.shape[-1]).permute(0, 2, 1, 3)


# ----------------------------------------------------------------------------- MoE router / dispatch
def _topk_lowest_index_first(x: torch.Tensor, k: int) -> tuple[torch.Tensor, torch.Tensor]:
    """top-k with ties resolved towards the lower index (the order ``jax.lax.top_k`` produces)."""
    idx = torch.argsort(x, dim=-1, descending=True, stable=True)[..., :k]
    return torch.gather(x, -1, idx), idx


def router_sigmoid_group(logits: torch.Tensor, bias: torch.Tensor, top_k: int, n_group: int, topk_group: int,
                         norm_topk_prob: bool, scaling: float):
    """DeepSeek-V3 routing (mintext/modules/moe.py:52-103): fp32 sigmoid scores; selection on scores + bias;
    group score = sum of the two best experts in a group; keep ``topk_group`` groups; global top-k among them;
    weights are the un-biased scores, optionally renormalised, times ``scaling``."""
    scores = torch.sigmoid(logits.float())
    sel = scores + bias.float()
    N, E = scores.shape
    per = E // n_group
    grouped = sel.view(N, n_group, per)
    gscore = _topk_lowest_index_first(grouped, min(2, per))[0].sum(-1)
    gidx = _topk_lowest_index_first(gscore, topk_group)[1]
    gmask = torch.zeros(N, n_group, dtype=torch.bool, device=logits.device).scatter_(1, gidx, True)
    emask = gmask.repeat_interleave(per, dim=1)
    masked = torch.where(emask, sel, torch.full_like(sel, float("-inf")))
    topk_idx = _topk_lowest_index_first(masked, top_k)[1]
    w = torch.gather(scores, 1, topk_idx)
    if norm_topk_prob:
        w = w / (w.sum(-1, keepdim=True) + 1e-20)
    return topk_idx, w * scaling, scores


def router_softmax_topk(logits: torch.Tensor, top_k: int, norm_topk_prob: bool, scaling: float = 1.0):
    """Qwen3-MoE style routing: fp32 softmax over experts, top-k, optional renormalisation.  Also returns the
    Switch-style load-balance auxiliary loss  E * sum_e f_e * P_e  (f_e = fraction of assignments routed to
    expert e, P_e = mean router probability of e)."""
    probs = torch.softmax(logits.float(), dim=-1)
    w, idx = _topk_lowest_index_first(probs, top_k)
    if norm_topk_prob:
        w = w / (w.sum(-1, keepdim=True) + 1e-20)
    N, E = probs.shape
    onehot = torch.zeros(N, E, device=logits.device, dtype=torch.float32).scatter_add_(
        1, idx, torch.ones_like(w, dtype=torch.float32))
    f = onehot.mean(0) / top_k
    aux = E * (f * probs.mean(0)).sum()
    return idx, w * scaling, probs, aux


def route(tokens: torch.Tensor, topk_idx: torch.Tensor, num_experts: int):
    """Capacity-free dispatch (mintext/kernels/moe_dispatch.py:47-81): each token is repeated K times, rows are
    ordered by expert with a stable sort (ties keep (token, slot) order).  Returns the permuted rows, the sort
    permutation and the per-expert row counts."""
    N, K = topk_idx.shape
    flat = topk_idx.reshape(-1)
    sort_idx = torch.argsort(flat, stable=True)
    rows = tokens.repeat_interleave(K, dim=0)[sort_idx]
    sizes = torch.bincount(flat, minlength=num_experts)
    return rows, sort_idx, sizes


def unroute(sorted_out: torch.Tensor, sort_idx: torch.Tensor, topk_w: torch.Tensor, K: int) -> torch.Tensor:
    """Inverse permutation then ``sum_k w[n,k] * y[n,k]`` (mintext/kernels/moe_dispatch.py:84-111)."""
    inv = torch.argsort(sort_idx)
    y = sorted_out[inv].view(-1, K, sorted_out.shape[-1])
    return torch.einsum("nkd,nk->nd", y, topk_w.to(y.dtype))


def grouped_matmul(x: torch.Tensor, w: torch.Tensor, group_sizes: torch.Tensor) -> torch.Tensor:
    """Ragged matmul: consecutive row groups of x times the matching ``w[e]`` (``[E,Kin,Kout]``)
    (mintext/kernels/grouped_matmul.py:58-76)."""
    out = x.new_zeros(x.shape[0], w.shape[-1])
    start = 0
    for e, n in enumerate(group_sizes.tolist()):
        if n:
            out[start:start + n] = x[start:start + n] @ w[e].to(x.dtype)
        start += n
    return out


def tgmm(lhs: torch.Tensor, rhs: torch.Tensor, group_sizes: torch.Tensor) -> torch.Tensor:
    """Per-expert ``lhs_e^T @ rhs_e`` -> ``[E,K,N]`` (mintext/kernels/grouped_matmul.py:197-235)."""
    E = group_sizes.numel()
    out = lhs.new_zeros(E, lhs.shape[1], rhs.shape[1])
    start = 0
    for e, n in enumerate(group_sizes.tolist()):
        if n:
            out[e] = lhs[start:start + n].t() @ rhs[start:start + n]
        start += n
    return out


# ----------------------------------------------------------------------------- gated delta rule
def causal_conv1d(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """Depth-wise causal conv: x ``[B,S,C]``, weight ``[C,1,K]`` (mintext/modules/linear_attention.py:17-40)."""
    K = weight.shape[-1]
    xt = F.pad(x.transpose(1, 2), (K - 1, 0))
    return F.conv1d(xt, weight.to(x.dtype), groups=x.shape[-1]).transpose(1, 2)


def l2_normalize(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    return x * torch.rsqrt((x * x).sum(-1, keepdim=True) + eps)


def chunk_gated_delta_rule(q, k, v, beta, g, chunk_size: int = 64, sequential: bool = False) -> torch.Tensor:
    """Chunked Gated Delta Rule in fp32 (mintext/modules/linear_attention.py:49-205).
    q,k ``[B,H,S,dk]``, v ``[B,H,S,dv]``, beta/g ``[B,H,S]`` -> ``[B,H,S,dv]``."""
    B, H, S, dk = q.shape
    dv = v.shape[-1]
    q = l2_normalize(q.float()) * dk ** -0.5
    k = l2_normalize(k.float())
    v, beta, g = v.float(), beta.float(), g.float()
    pad = (chunk_size - S % chunk_size) % chunk_size
    if pad:
        q, k, v = (F.pad(t, (0, 0, 0, pad)) for t in (q, k, v))
        beta, g = F.pad(beta, (0, pad)), F.pad(g, (0, pad))
    C = q.shape[2] // chunk_size
    L = chunk_size
    v_beta = (v * beta[..., None]).view(B, H, C, L, dv)
    k_beta = (k * beta[..., None]).view(B, H, C, L, dk)
    q, k, v = q.view(B, H, C, L, dk), k.view(B, H, C, L, dk), v.view(B, H, C, L, dv)
    g = g.view(B, H, C, L).cumsum(-1)
    tril = torch.tril(torch.ones(L, L, device=q.device))
    decay = torch.exp((g[..., :, None] - g[..., None, :]).clamp(-30.0, 30.0)) * tril
    attn = -(k_beta @ k.transpose(-1, -2)) * decay
    attn = attn.masked_fill(torch.triu(torch.ones(L, L, dtype=torch.bool, device=q.device)), 0.0)
    if sequential:
        # row-by-row forward substitution exactly as the reference loops it
        attn = attn.clone()
        for i in range(1, L):
            row = attn[..., i, :].clone()
            corr = torch.einsum("...j,...jk->...k", row, attn.clone())
            keep = (torch.arange(L, device=q.device) < i).to(corr.dtype)
            attn[..., i, :] = row + corr * keep
    else:
        # the loop above computes (I - attn)^-1 - I by forward substitution; solve it in one call
        eye = torch.eye(L, device=q.device)
        attn = torch.linalg.solve_triangular(eye - attn, eye.expand_as(attn).contiguous(), upper=False) - eye
    attn = attn + torch.eye(L, device=q.device)
    v_corr = attn @ v_beta
    g_exp = torch.exp(g.clamp(-30.0, 30.0))
    k_cumdecay = attn @ (k_beta * g_exp[..., None])
    g_last = g[..., -1:]
    k_decay = torch.exp((g_last[..., None] - g[..., None]).clamp(-30.0, 30.0))
    state = q.new_zeros(B, H, dk, dv)
    strict_upper = torch.triu(torch.ones(L, L, dtype=torch.bool, device=q.device), diagonal=1)
    outs = []
    for c in range(C):
        qc, kc = q[:, :, c], k[:, :, c]
        intra = (qc @ kc.transpose(-1, -2) * decay[:, :, c]).masked_fill(strict_upper, 0.0)
        v_prime = v_corr[:, :, c] - k_cumdecay[:, :, c] @ state
        inter = (qc @ state) * g_exp[:, :, c][..., None]
        outs.append(inter + intra @ v_prime)
        state = state * g_exp[:, :, c, -1][..., None, None] + (kc * k_decay[:, :, c]).transpose(-1, -2) @ v_prime
    out = torch.stack(outs, dim=2).reshape(B, H, C * L, dv)
    return out[:, :, :S]


def recurrent_gated_delta_rule(q, k, v, beta, g) -> torch.Tensor:
    """Token-by-token delta rule, the definition the chunked form must equal:
    ``S <- S * exp(g_t)``; ``S <- S + k_t (beta_t (v_t - S^T k_t))^T``; ``o_t = S^T q_t``."""
    B, H, S, dk = q.shape
    dv = v.shape[-1]
    q = l2_normalize(q.float()) * dk ** -0.5
    k = l2_normalize(k.float())
    v, beta, g = v.float(), beta.float(), g.float()
    state = q.new_zeros(B, H, dk, dv)
    outs = []
    for t in range(S):
        state = state * torch.exp(g[:, :, t])[..., None, None]
        kt, vt = k[:, :, t], v[:, :, t]
        pred = torch.einsum("bhkv,bhk->bhv", state, kt)
        delta = (vt - pred) * beta[:, :, t][..., None]
        state = state + kt[..., :, None] * delta[..., None, :]
        outs.append(torch.einsum("bhkv,bhk->bhv", state, q[:, :, t]))
    return torch.stack(outs, dim=2)


# ----------------------------------------------------------------------------- losses
def cross_entropy(logits: torch.Tensor, targets: torch.Tensor, label_smoothing: float = 0.0,
                  z_loss_weight: float = 0.0) -> tuple[torch.Tensor, torch.Tensor]:
    """Per-token loss and z-loss from fp32 log-softmax (mintext/trainer.py:83-194):
    ``(1-eps) * nll - eps * mean(log_softmax)`` and ``w * lse^2``; the returned loss already includes the
    z-loss term."""
    lf = logits.float()
    lse = torch.logsumexp(lf, dim=-1)
    logp = lf - lse[..., None]
    nll = -torch.gather(logp, -1, targets[..., None]).squeeze(-1)
    loss = (1.0 - label_smoothing) * nll - label_smoothing * logp.mean(-1) if label_smoothing > 0 else nll
    z = z_loss_weight * lse * lse
    return loss + z, z


# ----------------------------------------------------------------------------- optimizers
def adamw_update(p, g, m, v, step: int, lr: float, b1: float, b2: float, eps: float, wd: float):
    """optax.adamw: bias-corrected moments, ``p <- p - lr * (m_hat / (sqrt(v_hat) + eps) + wd * p)``."""
    m.mul_(b1).add_(g, alpha=1 - b1)
    v.mul_(b2).addcmul_(g, g, value=1 - b2)
    mh = m / (1 - b1 ** step)
    vh = v / (1 - b2 ** step)
    p.add_(mh / (vh.sqrt() + eps) + wd * p, alpha=-lr)


NS_COEFFS = (3.4445, -4.7750, 2.0315)


def newton_schulz(x: torch.Tensor, steps: int = 5, eps: float = 1e-8, coeffs=NS_COEFFS) -> torch.Tensor:
    """Quintic Newton-Schulz orthogonalisation of the last two dims (optax.contrib.muon):
    ``X <- a X + (b A + c A^2) X`` with ``A = X X^T``, applied on the wide orientation, after dividing by the
    Frobenius norm."""
    a, b, c = coeffs
    transposed = x.shape[-2] > x.shape[-1]
    if transposed:
        x = x.transpose(-1, -2)
    x = x / (x.norm(dim=(-2, -1), keepdim=True) + eps)
    for _ in range(steps):
        A = x @ x.transpose(-1, -2)
        x = a * x + (b * A + c * (A @ A)) @ x
    return x.transpose(-1, -2) if transposed else x


def newton_schulz_sliced(x: torch.Tensor, axis: int, all_reduce, steps: int = 5, eps: float = 1e-8,
                         coeffs=NS_COEFFS) -> torch.Tensor:
    """:func:`newton_schulz` for a matrix of which every rank of a group holds a slice: ``x`` ``[b, r, c]`` is the
    local slice, ``axis`` the sliced dimension (-2 rows, -1 columns) and ``all_reduce(t)`` sums ``t`` over the group in
    place.  The iteration is written on the Gram matrix of the *unsliced* dimension, which is a plain sum of the
    ranks' local Gram matrices (``X X^T = sum_l X_l X_l^T`` for column slices, ``X^T X`` for row slices); the
    polynomial then acts on each slice locally.  Equal to the whole-matrix iteration (``p(X X^T) X = X p(X^T X)``)."""
    a, b, c = coeffs
    ss = (x.float() ** 2).sum(dim=(-2, -1), keepdim=True)
    all_reduce(ss)
    x = x / (ss.sqrt() + eps)
    for _ in range(steps):
        if axis == -1:
            A = x @ x.transpose(-1, -2)
            all_reduce(A)
            x = a * x + (b * A + c * (A @ A)) @ x
        else:
            A = x.transpose(-1, -2) @ x
            all_reduce(A)
            x = a * x + x @ (b * A + c * (A @ A))
    return x
