"""Single-behaviour checks of modules and model families on the CPU / oracle path: one assertion family per test,
each against a value worked out by hand or by an independent few-line restatement of the math."""

import math

import pytest
import torch

from mintext_b200 import MinTextConfig
from mintext_b200.models import DecoderLayer, Transformer, make_causal_mask
from mintext_b200.modules import (MLP, Attention, Linear, MLAttention, MoEBlock, MoEExperts, MoERouter, RMSNorm,
                                  RotaryEmbedding, compute_inv_freq, make_sliding_window_mask)
from mintext_b200.modules.linear import ACT2FN
from mintext_b200.utils.pytree import count_params, estimate_param_count


def cfg(**kw):
    base = dict(dtype="float32", vocab_size=96, num_key_value_heads=2, num_hidden_layers=2, hidden_size=32,
                num_attention_heads=4, intermediate_size=64, seq_length=16)
    base.update(kw)
    return MinTextConfig(**base)


def gen(seed=0):
    return torch.Generator().manual_seed(seed)


def pos(B, S):
    return torch.arange(S)[None].expand(B, -1)


# ------------------------------------------------------------------ norm / linear
def test_rmsnorm_keeps_shape_and_dtype():
    n = RMSNorm(32, 1e-6, torch.float32)
    x = torch.randn(3, 5, 32)
    assert n(x).shape == x.shape and n(x).dtype == torch.float32


def test_rmsnorm_scale_parameter_multiplies_the_output():
    n = RMSNorm(16, 1e-6, torch.float32)
    x = torch.randn(4, 16)
    base = n(x)
    with torch.no_grad():
        n.scale.mul_(3.0)
    assert torch.allclose(n(x), 3.0 * base, atol=1e-6)


def test_rmsnorm_is_invariant_to_input_scale():
    n = RMSNorm(16, 1e-12, torch.float32)
    x = torch.randn(4, 16)
    assert torch.allclose(n(x), n(7.0 * x), atol=1e-5)


def test_linear_2d_kernel_is_a_plain_matmul():
    lin = Linear(8, 12, rngs=gen())
    x = torch.randn(5, 8)
    assert lin.kernel.shape == (8, 12) and torch.allclose(lin(x), x @ lin.kernel, atol=1e-6)


def test_linear_expanding_kernel_makes_heads():
    lin = Linear(8, (2, 6), rngs=gen())
    y = lin(torch.randn(3, 4, 8))
    assert lin.kernel.shape == (8, 2, 6) and y.shape == (3, 4, 2, 6)


def test_linear_contracting_kernel_consumes_heads():
    lin = Linear((2, 6), 8, rngs=gen())
    x = torch.randn(3, 4, 2, 6)
    want = torch.einsum("bshd,hde->bse", x, lin.kernel)
    assert lin.kernel.shape == (2, 6, 8) and torch.allclose(lin(x), want, atol=1e-5)


def test_linear_bias_is_added():
    lin = Linear(4, 6, use_bias=True, rngs=gen())
    with torch.no_grad():
        lin.bias.fill_(0.5)
    x = torch.zeros(2, 4)
    assert torch.allclose(lin(x), torch.full((2, 6), 0.5))


# ------------------------------------------------------------------ RoPE
def test_default_inverse_frequencies_follow_theta():
    inv, att = compute_inv_freq(cfg(rope_theta=10000.0), 8)
    want = torch.tensor([10000.0 ** (-2 * i / 8) for i in range(4)])
    assert att == 1.0 and torch.allclose(inv, want, rtol=1e-6)


def test_linear_rope_scaling_divides_every_frequency():
    base, _ = compute_inv_freq(cfg(), 16)
    lin, _ = compute_inv_freq(cfg(rope_type="linear", rope_scaling_factor=4.0), 16)
    assert torch.allclose(lin * 4.0, base)


def test_yarn_blends_between_scaled_and_unscaled_frequencies():
    c = cfg(rope_type="yarn", rope_scaling_factor=4.0, rope_original_max_position_embeddings=32, rope_theta=10000.0)
    base, _ = compute_inv_freq(cfg(rope_theta=10000.0), 32)
    y, _ = compute_inv_freq(c, 32)
    # every yarn frequency lies between the fully interpolated (base / factor) and the original value
    assert torch.all(y <= base * (1 + 1e-6)) and torch.all(y >= base / 4.0 * (1 - 1e-6))
    assert torch.allclose(y[0], base[0], rtol=1e-5)            # fastest dimension extrapolates (unchanged)
    assert torch.allclose(y[-1], base[-1] / 4.0, rtol=1e-5)    # slowest dimension is fully interpolated


def test_yarn_attention_factor_formula():
    _, att = compute_inv_freq(cfg(rope_type="yarn", rope_scaling_factor=8.0, rope_original_max_position_embeddings=32), 16)
    assert att == pytest.approx(0.1 * math.log(8.0) + 1.0)
    _, att1 = compute_inv_freq(cfg(rope_type="yarn", rope_scaling_factor=1.0, rope_original_max_position_embeddings=32), 16)
    assert att1 == pytest.approx(1.0)


def test_llama3_scaling_has_three_regions():
    c = cfg(rope_type="llama3", rope_scaling_factor=8.0, rope_original_max_position_embeddings=64, rope_theta=10000.0,
            rope_llama3_low_freq_factor=1.0, rope_llama3_high_freq_factor=4.0)
    base, _ = compute_inv_freq(cfg(rope_theta=10000.0), 64)
    l3, _ = compute_inv_freq(c, 64)
    wavelen = 2 * math.pi / base
    high = wavelen < 64 / 4.0          # short wavelengths: untouched
    low = wavelen > 64 / 1.0           # long wavelengths: divided by the factor
    assert high.any() and low.any()
    assert torch.allclose(l3[high], base[high]) and torch.allclose(l3[low], base[low] / 8.0)
    mid = ~(high | low)
    if mid.any():                      # smooth blend in between
        assert torch.all(l3[mid] < base[mid]) and torch.all(l3[mid] > base[mid] / 8.0)


def test_rope_is_a_rotation_of_dimension_pairs():
    c = cfg()
    rope = RotaryEmbedding(c)
    x = torch.randn(1, 5, 1, c.head_dim)
    y = rope(x, pos(1, 5))
    half = c.head_dim // 2
    inv, _ = compute_inv_freq(c, c.head_dim)
    ang = torch.arange(5)[:, None].float() * inv[None]
    want_first = x[0, :, 0, :half] * ang.cos() - x[0, :, 0, half:] * ang.sin()
    assert torch.allclose(y[0, :, 0, :half], want_first, atol=1e-5)


def test_rope_relative_property_of_scores():
    """<rope(q, m), rope(k, n)> depends on m - n only."""
    c = cfg()
    rope = RotaryEmbedding(c)
    q, k = torch.randn(1, 1, 1, c.head_dim), torch.randn(1, 1, 1, c.head_dim)
    def score(m, n):
        return float((rope(q, torch.tensor([[m]])) * rope(k, torch.tensor([[n]]))).sum())
    assert score(5, 2) == pytest.approx(score(9, 6), abs=1e-4)


def test_each_rope_variant_runs_through_attention():
    for kind, extra in (("linear", {}), ("yarn", {"rope_original_max_position_embeddings": 8}),
                        ("llama3", {"rope_original_max_position_embeddings": 8})):
        c = cfg(rope_type=kind, rope_scaling_factor=2.0, **extra)
        y = Attention(c, rngs=gen())(torch.randn(1, 16, 32), pos(1, 16))
        assert y.shape == (1, 16, 32) and torch.isfinite(y).all()


# ------------------------------------------------------------------ attention
def test_attention_head_counts_in_kernel_shapes():
    a = Attention(cfg(num_attention_heads=4, num_key_value_heads=2, head_dim=8), rngs=gen())
    assert a.query.kernel.shape == (32, 4, 8) and a.key.kernel.shape == (32, 2, 8) and a.out.kernel.shape == (4, 8, 32)


def test_mha_when_kv_heads_equal_heads():
    a = Attention(cfg(num_attention_heads=4, num_key_value_heads=4), rngs=gen())
    assert a.key.kernel.shape[1] == 4
    assert a(torch.randn(2, 6, 32), pos(2, 6)).shape == (2, 6, 32)


def test_qk_norm_adds_per_head_scales():
    a = Attention(cfg(use_qk_norm=True), rngs=gen(), use_qk_norm=True)
    assert a.q_norm.scale.shape == (cfg().head_dim,) and a.k_norm.scale.shape == (cfg().head_dim,)
    plain = Attention(cfg(), rngs=gen())
    assert not hasattr(plain, "q_norm")


def test_future_tokens_do_not_influence_the_past():
    a = Attention(cfg(), rngs=gen())
    x = torch.randn(1, 8, 32)
    y = a(x, pos(1, 8))
    x2 = x.clone()
    x2[0, 5:] += 1.0
    assert torch.allclose(a(x2, pos(1, 8))[0, :5], y[0, :5], atol=1e-5)


def test_sliding_window_limits_the_lookback():
    c = cfg()
    a = Attention(c, rngs=gen(), sliding_window=3)
    x = torch.randn(1, 10, 32)
    y = a(x, pos(1, 10))
    x2 = x.clone()
    x2[0, 0] += 5.0                     # token 0 is outside the window of tokens >= 3
    y2 = a(x2, pos(1, 10))
    assert torch.allclose(y2[0, 3:], y[0, 3:], atol=1e-5) and not torch.allclose(y2[0, 1], y[0, 1], atol=1e-5)


def test_causal_mask_is_lower_triangular():
    m = make_causal_mask(5)
    assert m.shape == (1, 1, 5, 5)
    upper = torch.triu(torch.ones(5, 5, dtype=torch.bool), 1)
    assert (m[0, 0][upper] < -1e9).all() and (m[0, 0][~upper] == 0).all()


def test_sliding_window_mask_shape_and_band():
    m = make_sliding_window_mask(6, 2)
    allowed = (m[0, 0] == 0)
    want = torch.tensor([[0 <= i - j < 2 for j in range(6)] for i in range(6)])
    assert m.shape == (1, 1, 6, 6) and torch.equal(allowed, want)


def test_attention_logit_softcap_bounds_the_effect_of_large_scores():
    c = cfg(attn_logit_softcapping=1.0)
    a = Attention(c, rngs=gen())
    x = torch.randn(1, 6, 32) * 50.0
    assert torch.isfinite(a(x, pos(1, 6))).all()


def test_query_pre_attn_scalar_sets_the_scale():
    a = Attention(cfg(query_pre_attn_scalar=64.0), rngs=gen())
    assert a.scale == pytest.approx(64.0 ** -0.5)
    b = Attention(cfg(), rngs=gen())
    assert b.scale == pytest.approx(cfg().head_dim ** -0.5)


# ------------------------------------------------------------------ MLA
def mla_cfg(**kw):
    base = dict(attention_type="mla", q_lora_rank=16, kv_lora_rank=12, qk_nope_head_dim=8, qk_rope_head_dim=4,
                v_head_dim=6)
    base.update(kw)
    return cfg(**base)


def test_mla_low_rank_projection_shapes():
    m = MLAttention(mla_cfg(), rngs=gen())
    assert m.q_a_proj.kernel.shape == (32, 16) and m.q_b_proj.kernel.shape == (16, 4, 12)
    assert m.kv_a_proj.kernel.shape == (32, 12 + 4) and m.kv_b_proj.kernel.shape == (12, 4, 8 + 6)
    assert m.out.kernel.shape == (4, 6, 32)


def test_mla_without_query_lora_projects_directly():
    m = MLAttention(mla_cfg(q_lora_rank=0), rngs=gen())
    assert hasattr(m, "q_proj") and not hasattr(m, "q_a_proj") and m.q_proj.kernel.shape == (32, 4, 12)


def test_mla_scale_uses_the_full_query_key_width():
    m = MLAttention(mla_cfg(), rngs=gen())
    assert m.scale == pytest.approx((8 + 4) ** -0.5)


def test_mla_output_is_finite_and_shaped():
    y = MLAttention(mla_cfg(), rngs=gen())(torch.randn(2, 7, 32), pos(2, 7))
    assert y.shape == (2, 7, 32) and torch.isfinite(y).all()


# ------------------------------------------------------------------ MLP / activations
def test_every_activation_name_resolves():
    for name in ("silu", "gelu", "gelu_pytorch_tanh", "relu"):
        assert callable(ACT2FN[name])
    x = torch.linspace(-2, 2, 9)
    assert torch.allclose(ACT2FN["relu"](x), x.clamp_min(0))
    assert torch.allclose(ACT2FN["silu"](x), x * torch.sigmoid(x))


def test_mlp_is_down_of_gated_product():
    m = MLP(cfg(), rngs=gen())
    x = torch.randn(3, 32)
    want = (torch.nn.functional.silu(x @ m.gate.kernel) * (x @ m.up.kernel)) @ m.down.kernel
    assert torch.allclose(m(x), want, atol=1e-5)


def test_mlp_with_tanh_gelu():
    m = MLP(cfg(hidden_activation="gelu_pytorch_tanh"), rngs=gen())
    x = torch.randn(3, 32)
    want = (torch.nn.functional.gelu(x @ m.gate.kernel, approximate="tanh") * (x @ m.up.kernel)) @ m.down.kernel
    assert torch.allclose(m(x), want, atol=1e-5)


# ------------------------------------------------------------------ MoE
def moe_cfg(**kw):
    base = dict(model_type="deepseek_v3", num_experts=8, num_experts_per_tok=2, moe_intermediate_size=16, n_group=4,
                topk_group=2, first_k_dense_replace=1, n_shared_experts=1)
    base.update(kw)
    return cfg(**base)


def test_router_outputs_have_the_documented_shapes():
    r = MoERouter(moe_cfg(), rngs=gen())
    idx, w, scores = r(torch.randn(10, 32))
    assert idx.shape == (10, 2) and w.shape == (10, 2) and scores.shape == (10, 8)


def test_router_indices_are_distinct_and_in_range():
    r = MoERouter(moe_cfg(), rngs=gen())
    idx, _, _ = r(torch.randn(50, 32))
    assert int(idx.min()) >= 0 and int(idx.max()) < 8 and bool((idx[:, 0] != idx[:, 1]).all())


def test_router_weights_are_normalised_and_scaled():
    r = MoERouter(moe_cfg(routed_scaling_factor=2.5, norm_topk_prob=True), rngs=gen())
    _, w, _ = r(torch.randn(20, 32))
    assert torch.allclose(w.sum(-1), torch.full((20,), 2.5), atol=1e-4)


def test_selection_bias_steers_choice_but_not_weights():
    r = MoERouter(moe_cfg(n_group=1, topk_group=1), rngs=gen())
    x = torch.randn(30, 32)
    _, _, scores = r(x)
    with torch.no_grad():
        r.e_score_correction_bias[3] = 100.0
    idx, w, _ = r(x)
    assert bool((idx == 3).any(dim=-1).all())                          # expert 3 is always picked
    picked = scores.gather(1, idx)
    assert torch.allclose(w / w.sum(-1, keepdim=True), picked / picked.sum(-1, keepdim=True), atol=1e-5)


def test_group_limited_routing_stays_inside_the_best_groups():
    c = moe_cfg(n_group=4, topk_group=1, num_experts_per_tok=2)
    r = MoERouter(c, rngs=gen())
    idx, _, _ = r(torch.randn(40, 32))
    assert bool((idx[:, 0] // 2 == idx[:, 1] // 2).all())              # both picks from one group of two experts


def test_experts_output_shape_and_zero_weight_gives_zero():
    c = moe_cfg()
    e = MoEExperts(c, rngs=gen())
    x = torch.randn(6, 32)
    idx = torch.randint(0, 8, (6, 2))
    y = e(x, idx, torch.zeros(6, 2))
    assert y.shape == (6, 32) and torch.count_nonzero(y) == 0


def test_moe_block_adds_the_shared_expert():
    blk = MoEBlock(moe_cfg(), rngs=gen())
    x = torch.randn(2, 5, 32)
    out, aux = blk(x)
    routed = blk.experts(x.reshape(10, 32), aux["topk_indices"], blk.router(x.reshape(10, 32))[1]).reshape(2, 5, 32)
    assert torch.allclose(out, routed + blk.shared_expert(x), atol=1e-5)
    assert aux["topk_indices"].shape == (10, 2) and aux["scores"].shape == (10, 8)


def test_moe_layers_start_after_the_dense_prefix():
    c = moe_cfg(num_hidden_layers=3, first_k_dense_replace=2)
    kinds = [type(DecoderLayer(c, i, rngs=gen()).mlp).__name__ for i in range(3)]
    assert kinds == ["MLP", "MLP", "MoEBlock"]


def test_model_returns_one_aux_entry_per_layer_with_none_for_dense():
    c = moe_cfg(num_hidden_layers=3)
    _, aux = Transformer(c, rngs=0)(torch.randint(0, 96, (1, 8)), pos(1, 8))
    assert len(aux) == 3 and aux[0] is None and aux[1] is not None and "topk_indices" in aux[1]


# ------------------------------------------------------------------ decoder layer / transformer
def test_decoder_layer_preserves_shape():
    y, aux = DecoderLayer(cfg(), 0, rngs=gen())(torch.randn(2, 6, 32), pos(2, 6))
    assert y.shape == (2, 6, 32) and aux is None


def test_four_norm_layer_has_post_norms():
    layer = DecoderLayer(cfg(use_post_ffw_norm=True), 0, rngs=gen())
    assert hasattr(layer, "pre_ffw_norm") and hasattr(layer, "post_ffw_norm")
    assert not hasattr(DecoderLayer(cfg(), 0, rngs=gen()), "post_ffw_norm")
    assert layer(torch.randn(1, 4, 32), pos(1, 4))[0].shape == (1, 4, 32)


def test_logits_shape():
    logits, _ = Transformer(cfg(), rngs=0)(torch.randint(0, 96, (2, 8)), pos(2, 8))
    assert logits.shape == (2, 8, 96)


def test_tied_embeddings_have_no_separate_head():
    tied = Transformer(cfg(tie_word_embeddings=True), rngs=0)
    untied = Transformer(cfg(tie_word_embeddings=False), rngs=0)
    assert not hasattr(tied, "output_proj") and hasattr(untied, "output_proj")
    assert count_params(untied) - count_params(tied) == 96 * 32


def test_parameter_count_matches_the_closed_form():
    c = cfg(tie_word_embeddings=False)
    m = Transformer(c, rngs=0)
    D, V, H, Hkv, dh, M, L = 32, 96, 4, 2, c.head_dim, 64, 2
    per_layer = D * (H + 2 * Hkv) * dh + H * dh * D + 3 * D * M + 2 * D      # projections + MLP + two norm scales
    assert count_params(m) == 2 * V * D + L * per_layer + D
    assert abs(estimate_param_count(c) - count_params(m)) <= L * 2 * D + D  # the estimate ignores norm scales


def test_embedding_scale_is_sqrt_hidden():
    c = cfg(scale_embeddings=True)
    assert Transformer(c, rngs=0).embedding_scale == pytest.approx(math.sqrt(32))
    assert Transformer(cfg(), rngs=0).embedding_scale is None


def test_final_logit_softcap_bounds_logits():
    c = cfg(final_logit_softcapping=2.0)
    m = Transformer(c, rngs=0)
    with torch.no_grad():
        m.token_embedder.mul_(50.0)
    logits, _ = m(torch.randint(0, 96, (1, 8)), pos(1, 8))
    assert float(logits.detach().abs().max()) <= 2.0


def test_gradients_reach_every_trainable_parameter():
    c = cfg(model_type="gemma3", use_qk_norm=True, use_post_ffw_norm=True, scale_embeddings=True, sliding_window=4,
            sliding_window_pattern=2, tie_word_embeddings=True)
    m = Transformer(c, rngs=0)
    logits, _ = m(torch.randint(0, 96, (1, 8)), pos(1, 8))
    logits.square().mean().backward()
    missing = [n for n, p in m.named_parameters() if p.requires_grad and (p.grad is None or not torch.isfinite(p.grad).all())]
    assert not missing, missing


def test_explicit_causal_mask_equals_the_builtin_causality():
    m = Transformer(cfg(), rngs=0)
    tok = torch.randint(0, 96, (1, 8))
    a, _ = m(tok, pos(1, 8))
    b, _ = m(tok, pos(1, 8), mask=make_causal_mask(8))
    assert torch.allclose(a, b, atol=1e-4)


# ------------------------------------------------------------------ layer-type patterns
def test_gemma3_default_pattern_is_five_local_one_global():
    t = MinTextConfig(model_type="gemma3", num_hidden_layers=12).layer_types
    assert [i for i, k in enumerate(t) if k == "full_attention"] == [5, 11]


def test_gemma3_custom_pattern():
    t = MinTextConfig(model_type="gemma3", num_hidden_layers=6, sliding_window_pattern=3).layer_types
    assert t == ["sliding_attention", "sliding_attention", "full_attention"] * 2


def test_gemma3_local_layers_use_the_local_rope_base():
    c = cfg(model_type="gemma3", num_hidden_layers=2, sliding_window=4, sliding_window_pattern=2, rope_theta=1e6,
            rope_local_theta=1e4)
    m = Transformer(c, rngs=0)
    local, glob = m.layers[0].attention.rope, m.layers[1].attention.rope
    assert float(local._inv_freq[-1]) > float(glob._inv_freq[-1])      # smaller base -> faster slowest frequency


def test_qwen3_next_interval_places_full_attention():
    t = MinTextConfig(model_type="qwen3_next", num_hidden_layers=8, full_attention_interval=4).layer_types
    assert [i for i, k in enumerate(t) if k == "full_attention"] == [3, 7]


def test_qwen3_window_layers_come_first():
    t = MinTextConfig(model_type="qwen3", num_hidden_layers=4, use_sliding_window=True, max_window_layers=3).layer_types
    assert t.count("sliding_attention") == 3 and t[-1] == "full_attention"


# ------------------------------------------------------------------ named activations for remat
def test_projection_outputs_carry_remat_names():
    a = Attention(cfg(), rngs=gen())
    assert (a.query.remat_name, a.key.remat_name, a.value.remat_name, a.out.remat_name) == \
        ("query_proj", "key_proj", "value_proj", "out_proj")
    m = MLP(cfg(), rngs=gen())
    assert {m.gate.remat_name, m.up.remat_name, m.down.remat_name} == {"mlp_gate_proj", "mlp_up", "mlp_down"}


@pytest.mark.parametrize("policy", ["save_qkv_proj", "save_dot_except_mlp", "qkv_proj_offloaded", "minimal_offloaded"])
def test_remat_policy_keeps_the_loss(policy):
    tok = torch.randint(0, 96, (2, 8))
    out = []
    for pol in ("none", policy):
        m = Transformer(cfg(remat_policy=pol), rngs=0)
        logits, _ = m(tok, pos(2, 8))
        out.append(logits)
    assert torch.allclose(out[0], out[1], atol=1e-5)
