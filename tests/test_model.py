"""Modules and models on the CPU / oracle path (mirrors the reference's tests/test_model.py)."""

import math

import pytest
import torch

from mintext_b200 import MinTextConfig
from mintext_b200.models import DecoderLayer, Transformer, make_causal_mask
from mintext_b200.modules import (MLP, Attention, GatedDeltaRuleAttention, Linear, MLAttention, MoEBlock, MoEExperts,
                                  MoERouter, RMSNorm, RotaryEmbedding, compute_inv_freq, make_sliding_window_mask)
from mintext_b200.ops import oracle


def cfg(**kw):
    base = dict(dtype="float32", vocab_size=128, num_key_value_heads=2)
    base.update(kw)
    return MinTextConfig(**base)


def gen(seed=0):
    return torch.Generator().manual_seed(seed)


def positions(B, S):
    return torch.arange(S)[None].expand(B, -1)


# ------------------------------------------------------------------ basic modules
def test_rmsnorm_unit_rms():
    n = RMSNorm(64, 1e-5, torch.float32)
    y = n(torch.randn(4, 10, 64) * 3)
    assert torch.allclose(y.pow(2).mean(-1).sqrt(), torch.ones(4, 10), atol=1e-3)


def test_linear_three_kernel_shapes():
    g = gen()
    x = torch.randn(2, 5, 16)
    assert Linear(16, 32, rngs=g)(x).shape == (2, 5, 32)
    expand = Linear(16, (4, 8), rngs=g)
    assert expand.kernel.shape == (16, 4, 8) and expand(x).shape == (2, 5, 4, 8)
    contract = Linear((4, 8), 16, rngs=g)
    assert contract.kernel.shape == (4, 8, 16) and contract(torch.randn(2, 5, 4, 8)).shape == (2, 5, 16)
    b = Linear(16, 8, use_bias=True, rngs=g)
    assert b.bias is not None and b(x).shape == (2, 5, 8)


def test_linear_init_scale():
    w = Linear(1024, 256, rngs=gen()).kernel
    assert abs(w.std().item() * math.sqrt(1024) - 0.88) < 0.05  # truncated normal(+-2 sigma) has std ~0.88
    assert w.abs().max().item() <= 2.0 / math.sqrt(1024) + 1e-6


# ------------------------------------------------------------------ rope
def test_rope_identity_at_position_zero_and_norm_preserved():
    c = cfg()
    rope = RotaryEmbedding(c)
    x = torch.randn(2, 6, 4, c.head_dim)
    y0 = rope(x, torch.zeros(2, 6, dtype=torch.long))
    assert torch.allclose(y0, x, atol=1e-6)
    y = rope(x, positions(2, 6))
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1), atol=1e-4)


def test_rope_variants():
    base, _ = compute_inv_freq(cfg(), 32)
    lin, _ = compute_inv_freq(cfg(rope_type="linear", rope_scaling_factor=2.0), 32)
    assert torch.allclose(lin, base / 2)
    _, att = compute_inv_freq(cfg(rope_type="yarn", rope_scaling_factor=4.0, rope_original_max_position_embeddings=64), 32)
    assert att == pytest.approx(0.1 * math.log(4.0) + 1.0)
    l3, _ = compute_inv_freq(cfg(rope_type="llama3", rope_scaling_factor=8.0, rope_original_max_position_embeddings=64,
                                 rope_theta=10000.0), 32)
    assert torch.allclose(l3[0], base[0]) and l3[-1] < base[-1]  # high freq kept, low freq scaled down
    assert cfg(rope_type="llama3_1").rope_type == "llama3"


def test_rope_partial_and_interleave():
    c = cfg(partial_rotary_factor=0.5)
    rope = RotaryEmbedding(c)
    x = torch.randn(1, 4, 2, c.head_dim)
    y = rope(x, positions(1, 4))
    assert torch.equal(y[..., c.head_dim // 2:], x[..., c.head_dim // 2:])
    ci = cfg(rope_interleave=True)
    yi = RotaryEmbedding(ci)(x, positions(1, 4))
    assert yi.shape == x.shape and not torch.allclose(yi, x)


# ------------------------------------------------------------------ attention
def test_attention_shape_and_gqa_equals_repeated_kv():
    c = cfg(num_attention_heads=4, num_key_value_heads=2)
    attn = Attention(c, rngs=gen())
    x = torch.randn(2, 16, c.hidden_size)
    out = attn(x, positions(2, 16))
    assert out.shape == x.shape
    q = torch.randn(2, 16, 4, 8)
    k = torch.randn(2, 16, 2, 8)
    v = torch.randn(2, 16, 2, 8)
    a = oracle.attention(q, k, v, 8 ** -0.5)
    b = oracle.attention(q, k.repeat_interleave(2, 2), v.repeat_interleave(2, 2), 8 ** -0.5)
    assert torch.allclose(a, b, atol=1e-5)


def test_attention_is_causal():
    c = cfg()
    attn = Attention(c, rngs=gen())
    x = torch.randn(1, 12, c.hidden_size)
    y1 = attn(x, positions(1, 12))
    x2 = x.clone()
    x2[:, 8:] += 1.0
    y2 = attn(x2, positions(1, 12))
    assert torch.allclose(y1[:, :8], y2[:, :8], atol=1e-5)


def test_attention_qk_norm_window_gate_and_mask_path():
    c = cfg()
    x = torch.randn(1, 12, c.hidden_size)
    a = Attention(c, rngs=gen(), use_qk_norm=True, sliding_window=4, use_gate=True)
    assert a.query.kernel.shape == (c.hidden_size, 4, 2 * c.head_dim)
    y = a(x, positions(1, 12))
    ym = a(x, positions(1, 12), make_causal_mask(12))
    assert torch.allclose(y, ym, atol=1e-5)


def test_sliding_window_mask_semantics():
    m = make_sliding_window_mask(6, 3)[0, 0]
    allowed = m == 0
    for i in range(6):
        for j in range(6):
            assert bool(allowed[i, j]) == (0 <= i - j < 3)


def test_mla_with_and_without_q_lora():
    for q_lora in (0, 16):
        c = cfg(attention_type="mla", q_lora_rank=q_lora, kv_lora_rank=16, qk_nope_head_dim=8, qk_rope_head_dim=4,
                v_head_dim=8)
        m = MLAttention(c, 0, rngs=gen())
        x = torch.randn(2, 10, c.hidden_size)
        assert m(x, positions(2, 10)).shape == x.shape
        assert hasattr(m, "q_a_proj") == (q_lora > 0)
        # causal by default; the compat switch reproduces the reference's unmasked behaviour
        x2 = x.clone()
        x2[:, 6:] += 1
        assert torch.allclose(m(x, positions(2, 10))[:, :6], m(x2, positions(2, 10))[:, :6], atol=1e-5)
    nc = MLAttention(cfg(attention_type="mla", kv_lora_rank=16, qk_nope_head_dim=8, qk_rope_head_dim=4, v_head_dim=8,
                         attention_causal_mla=False), 0, rngs=gen())
    assert not torch.allclose(nc(x, positions(2, 10))[:, :6], nc(x2, positions(2, 10))[:, :6], atol=1e-5)


# ------------------------------------------------------------------ MLP / MoE
@pytest.mark.parametrize("act", ["silu", "gelu", "gelu_pytorch_tanh", "relu"])
def test_mlp_activations(act):
    c = cfg(hidden_activation=act)
    assert MLP(c, rngs=gen())(torch.randn(2, 5, c.hidden_size)).shape == (2, 5, c.hidden_size)


def moe_cfg(**kw):
    base = dict(num_experts=8, num_experts_per_tok=2, moe_intermediate_size=32, n_group=4, topk_group=2,
                first_k_dense_replace=1, n_shared_experts=1)
    base.update(kw)
    return cfg(**base)


def test_router_shapes_ranges_bias():
    c = moe_cfg()
    r = MoERouter(c, rngs=gen())
    x = torch.randn(20, c.hidden_size)
    idx, w, scores = r(x)
    assert idx.shape == (20, 2) and w.shape == (20, 2) and scores.shape == (20, 8)
    assert (scores >= 0).all() and (scores <= 1).all() and idx.max() < 8
    assert torch.allclose(w.sum(-1), torch.full((20,), c.routed_scaling_factor), atol=1e-4)
    r.e_score_correction_bias.data[3] = 100.0  # the bias steers selection, not the weights
    idx2, w2, _ = r(x)
    assert (idx2 == 3).any(dim=-1).all()
    sel = scores.gather(1, idx2)
    assert torch.allclose(w2, sel / sel.sum(-1, keepdim=True) * c.routed_scaling_factor, atol=1e-5)


def test_softmax_router_and_aux_loss():
    c = moe_cfg(router_type="softmax_topk", n_group=1, topk_group=1)
    r = MoERouter(c, rngs=gen())
    idx, w, probs = r(torch.randn(50, c.hidden_size))
    assert torch.allclose(probs.sum(-1), torch.ones(50), atol=1e-5)
    assert r.last_aux_loss is not None and r.last_aux_loss.item() >= 0.99  # >= 1 with equality iff balanced


def test_experts_and_block_aux():
    c = moe_cfg()
    blk = MoEBlock(c, rngs=gen())
    x = torch.randn(2, 6, c.hidden_size)
    out, aux = blk(x)
    assert out.shape == x.shape and aux["topk_indices"].shape == (12, 2) and aux["scores"].shape == (12, 8)
    ex = MoEExperts(c, rngs=gen())
    assert ex.gate_up_proj.shape == (8, c.hidden_size, 64) and ex.down_proj.shape == (8, 32, c.hidden_size)
    # against a per-token loop
    flat = x.reshape(12, -1)
    idx, w, _ = blk.router(flat)
    got = blk.experts(flat, idx, w)
    ref = torch.zeros_like(flat)
    for n in range(12):
        for k in range(2):
            e = idx[n, k]
            h = flat[n] @ blk.experts.gate_up_proj[e]
            h = torch.nn.functional.silu(h[:32]) * h[32:]
            ref[n] += w[n, k] * (h @ blk.experts.down_proj[e])
    assert torch.allclose(got, ref, atol=1e-5)


# ------------------------------------------------------------------ GDN
def test_gdn_module_and_chunk_equals_recurrence():
    c = cfg(model_type="qwen3_next", linear_key_head_dim=8, linear_value_head_dim=8, linear_num_key_heads=2,
            linear_num_value_heads=4)
    g = GatedDeltaRuleAttention(c, rngs=gen())
    x = torch.randn(2, 70, c.hidden_size)
    y = g(x)
    assert y.shape == x.shape and torch.isfinite(y).all()
    q, k = torch.randn(1, 2, 130, 8), torch.randn(1, 2, 130, 8)
    v, beta, gg = torch.randn(1, 2, 130, 12), torch.rand(1, 2, 130), -torch.rand(1, 2, 130)
    a = oracle.chunk_gated_delta_rule(q, k, v, beta, gg)
    b = oracle.recurrent_gated_delta_rule(q, k, v, beta, gg)
    s = oracle.chunk_gated_delta_rule(q, k, v, beta, gg, sequential=True)
    assert torch.allclose(a, b, atol=1e-4) and torch.allclose(a, s, atol=1e-5)


# ------------------------------------------------------------------ layers / models
def test_decoder_layer_and_hybrid_placement():
    c = cfg(model_type="qwen3_next", num_hidden_layers=4, full_attention_interval=2, linear_key_head_dim=8,
            linear_value_head_dim=8, use_qk_norm=True)
    kinds = [type(DecoderLayer(c, i, rngs=gen()).attention).__name__ for i in range(4)]
    assert kinds == ["GatedDeltaRuleAttention", "Attention", "GatedDeltaRuleAttention", "Attention"]
    d = cfg(model_type="deepseek_v3", num_hidden_layers=3, **{k: v for k, v in moe_cfg().model_dump().items()
                                                             if k in ("num_experts", "num_experts_per_tok", "moe_intermediate_size", "n_group", "topk_group", "first_k_dense_replace")})
    has = [DecoderLayer(d, i, rngs=gen()).has_moe for i in range(3)]
    assert has == [False, True, True]


FAMILIES = {
    "llama3": dict(),
    "qwen3": dict(use_qk_norm=True, use_sliding_window=True, sliding_window=8, max_window_layers=1),
    "deepseek_v3": dict(attention_type="mla", q_lora_rank=16, kv_lora_rank=16, qk_nope_head_dim=8, qk_rope_head_dim=4,
                        v_head_dim=8, num_experts=8, num_experts_per_tok=2, moe_intermediate_size=32, n_group=4,
                        topk_group=2, first_k_dense_replace=1),
    "qwen3_next": dict(use_qk_norm=True, full_attention_interval=2, partial_rotary_factor=0.25, linear_key_head_dim=8,
                       linear_value_head_dim=8, num_experts=4, num_experts_per_tok=2, moe_intermediate_size=32,
                       n_group=1, topk_group=1, first_k_dense_replace=0),
    "gemma3": dict(use_qk_norm=True, query_pre_attn_scalar=32.0, attn_logit_softcapping=50.0,
                   final_logit_softcapping=30.0, use_post_ffw_norm=True, scale_embeddings=True, sliding_window=8,
                   sliding_window_pattern=2, hidden_activation="gelu_pytorch_tanh", tie_word_embeddings=True),
}


@pytest.mark.parametrize("family", list(FAMILIES))
def test_forward_and_grad_per_family(family):
    c = cfg(model_type=family, num_hidden_layers=2, **FAMILIES[family])
    m = Transformer(c, rngs=0)
    tok = torch.randint(0, c.vocab_size, (2, 16))
    logits, aux = m(tok, positions(2, 16))
    assert logits.shape == (2, 16, c.vocab_size) and len(aux) == 2 and torch.isfinite(logits).all()
    logits.float().mean().backward()
    grads = [p.grad for p in m.parameters() if p.requires_grad]
    assert all(g is not None for g in grads)
    if c.final_logit_softcapping:
        assert logits.abs().max() <= c.final_logit_softcapping


def test_transformer_tie_hidden_and_mask():
    c = cfg(tie_word_embeddings=True)
    m = Transformer(c, rngs=0)
    assert not hasattr(m, "output_proj")
    tok = torch.randint(0, c.vocab_size, (2, 8))
    hidden, _ = m(tok, positions(2, 8), return_hidden=True)
    assert hidden.shape == (2, 8, c.hidden_size)
    a, _ = m(tok, positions(2, 8))
    b, _ = m(tok, positions(2, 8), make_causal_mask(8))
    assert torch.allclose(a, b, atol=1e-5)
    assert make_causal_mask(4).shape == (1, 1, 4, 4)


def test_gemma_embedding_scale_rounds_in_compute_dtype():
    c = MinTextConfig(model_type="gemma3", hidden_size=2560, num_attention_heads=8, head_dim=32, scale_embeddings=True,
                      vocab_size=16, num_hidden_layers=1, intermediate_size=64)
    m = Transformer(c, rngs=0)
    tok = torch.zeros(1, 1, dtype=torch.long)
    from mintext_b200.ops import functional as F

    x = F.embedding(m.token_embedder, tok, torch.bfloat16, m.embedding_scale)
    expect = m.token_embedder[0].to(torch.bfloat16) * torch.tensor(50.5, dtype=torch.bfloat16)
    assert torch.equal(x[0, 0], expect)


@pytest.mark.parametrize("policy", ["none", "full", "minimal", "save_qkv_proj", "save_dot_except_mlp",
                                    "qkv_proj_offloaded", "minimal_offloaded"])
def test_every_remat_policy_gives_the_same_gradients(policy):
    tok = torch.randint(0, 128, (2, 12))
    ref = None
    for pol in ("none", policy):
        m = Transformer(cfg(remat_policy=pol), rngs=0)
        logits, _ = m(tok, positions(2, 12))
        logits.pow(2).mean().backward()
        g = torch.cat([p.grad.reshape(-1) for p in m.parameters()])
        if ref is None:
            ref = g
        else:
            assert torch.allclose(g, ref, atol=1e-6)


def test_fp8_matmul_correlates_with_exact():
    from mintext_b200.modules.linear import fp8_matmul_reference

    x, w = torch.randn(64, 128), torch.randn(128, 96) * 0.05
    a = fp8_matmul_reference(x, w, torch.float32)
    b = x @ w
    corr = torch.corrcoef(torch.stack([a.reshape(-1), b.reshape(-1)]))[0, 1]
    assert corr > 0.95
    c = cfg(use_fp8=True)
    assert torch.isfinite(MLP(c, rngs=gen())(torch.randn(2, 4, c.hidden_size))).all()


def test_mxfp8_matmul_reference_is_close_to_exact():
    """Block scaling (one power-of-two scale per 32 elements) keeps the product within a few percent even when
    the columns of the activation differ by orders of magnitude, where one per-tensor scale would flush them."""
    from mintext_b200.modules.linear import mxfp8_matmul_reference

    x = torch.randn(64, 128) * torch.logspace(-3, 2, 128)
    w = torch.randn(128, 96) * 0.05
    a = mxfp8_matmul_reference(x, w, torch.float32)
    b = x @ w
    assert ((a - b).norm() / b.norm()).item() < 0.05
    c = cfg(use_fp8=True, fp8_recipe="mx_block")
    assert torch.isfinite(MLP(c, rngs=gen())(torch.randn(2, 4, c.hidden_size))).all()
