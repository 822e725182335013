"""Losses, schedules, optimizers, train / eval steps, gradient accumulation (mirrors tests/test_train_step.py)."""

import math

import pytest
import torch

from mintext_b200 import MinTextConfig, trainer
from mintext_b200.models import Transformer
from mintext_b200.optim import accumulate_gradients, create_lr_schedule, create_optimizer
from mintext_b200.optim.optimizer import muon_matrix_view, weight_decay_mask
from mintext_b200.ops import oracle


def cfg(**kw):
    base = dict(dtype="float32", vocab_size=64, num_key_value_heads=2, steps=20)
    base.update(kw)
    return MinTextConfig(**base)


def make_batch(c, B=4, S=16, seed=0):
    g = torch.Generator().manual_seed(seed)
    t = torch.randint(0, c.vocab_size, (B, S), generator=g)
    return {"input_tokens": t, "target_tokens": t}


# ---------------------------------------------------------------- cross entropy
def test_ce_shape_positive_perfect():
    logits = torch.randn(2, 5, 11)
    tgt = torch.randint(0, 11, (2, 5))
    loss, z = trainer.cross_entropy_loss(logits, tgt)
    assert loss.shape == (2, 5) and (loss > 0).all() and float(z.abs().sum()) == 0
    perfect = torch.full((1, 3, 7), -30.0)
    t = torch.tensor([[1, 2, 3]])
    perfect.scatter_(2, t[..., None], 30.0)
    assert trainer.cross_entropy_loss(perfect, t)[0].max() < 1e-6


def test_ce_label_smoothing_and_zloss_match_dense_formula():
    logits = torch.randn(3, 4, 9, requires_grad=True)
    tgt = torch.randint(0, 9, (3, 4))
    ls, zw = 0.1, 1e-2
    loss, z = trainer.cross_entropy_with_z_loss(logits, tgt, ls, zw)
    logp = torch.log_softmax(logits, -1)
    onehot = torch.nn.functional.one_hot(tgt, 9).float()
    soft = onehot * (1 - ls) + ls / 9
    lse = torch.logsumexp(logits, -1)
    assert torch.allclose(loss, -(soft * logp).sum(-1) + zw * lse ** 2, atol=1e-5)
    assert torch.allclose(z, zw * lse ** 2, atol=1e-6)
    # gradient: probs * (1 + 2 w lse) - ls/V - (1 - ls) onehot
    loss.sum().backward()
    probs = torch.softmax(logits.detach(), -1)
    want = probs * (1 + 2 * zw * lse.detach()[..., None]) - ls / 9 - (1 - ls) * onehot
    assert torch.allclose(logits.grad, want, atol=1e-5)


def test_chunked_ce_equals_full():
    h = torch.randn(24, 16)
    w = torch.randn(16, 30)
    tgt = torch.randint(0, 30, (24,))
    full, zf = trainer.cross_entropy_loss(h @ w, tgt, 0.05, 1e-3)
    ch, zc = trainer.chunked_cross_entropy_loss(h, tgt, lambda x: x @ w, 4, 0.05, 1e-3)
    assert torch.allclose(full, ch, atol=1e-5) and torch.allclose(zf, zc, atol=1e-6)


def test_compute_loss_with_vocab_tiles_matches_plain():
    c1, c2 = cfg(per_device_batch_size=4, seq_length=16), cfg(per_device_batch_size=4, seq_length=16, num_vocab_tiles=4)
    m = Transformer(c1, rngs=0)
    b = make_batch(c1)
    l1, a1 = trainer.compute_loss(None, m, c1, b)
    l2, a2 = trainer.compute_loss(None, m, c2, b)
    assert torch.allclose(l1, l2, atol=1e-5) and a1["per_token_loss"].shape == (4, 16)


# ---------------------------------------------------------------- schedules
def test_cosine_linear_and_wsd_schedules():
    c = cfg(steps=100, learning_rate=1.0, warmup_steps_fraction=0.1, lr_final_fraction=0.1)
    s = create_lr_schedule(c)
    assert s(0) == 0 and s(5) == pytest.approx(0.5) and s(10) == pytest.approx(1.0)
    assert s(100) == pytest.approx(0.1) and s(55) == pytest.approx(0.1 + 0.9 * 0.5 * (1 + math.cos(math.pi * 0.5)))
    lin = create_lr_schedule(cfg(steps=100, learning_rate=1.0, lr_schedule="linear"))
    assert lin(55) == pytest.approx(0.55) and lin(100) == pytest.approx(0.1)
    w = create_lr_schedule(cfg(steps=100, learning_rate=1.0, lr_schedule="wsd", wsd_decay_steps_fraction=0.2))
    assert w(5) == pytest.approx(0.5) and w(50) == 1.0 and w(79) == 1.0 and w(90) == pytest.approx(0.55)
    assert w(100) == pytest.approx(0.1)
    wc = create_lr_schedule(cfg(steps=100, learning_rate=1.0, lr_schedule="wsd", wsd_decay_style="cosine"))
    assert wc(95) == pytest.approx(0.1 + 0.9 * 0.5)
    assert create_lr_schedule(cfg(steps=3, learning_rate=1.0))(1) == pytest.approx(1.0)  # warm-up is at least 1 step


# ---------------------------------------------------------------- optimizers
def test_weight_decay_mask_and_muon_views():
    assert weight_decay_mask("layers.0.pre_attn_norm.scale") and weight_decay_mask("token_embedder")
    assert not weight_decay_mask("layers.1.mlp.router.e_score_correction_bias")
    assert muon_matrix_view("layers.0.mlp.gate.kernel", (8, 16)) == (1, 8, 16)
    assert muon_matrix_view("layers.0.attention.query.kernel", (8, 2, 4)) == (1, 8, 8)
    assert muon_matrix_view("layers.0.attention.out.kernel", (2, 4, 8)) == (1, 8, 8)
    assert muon_matrix_view("layers.0.mlp.experts.gate_up_proj", (4, 8, 16)) == (4, 8, 16)
    assert muon_matrix_view("token_embedder", (64, 8)) is None and muon_matrix_view("final_norm.scale", (8,)) is None


def test_adamw_matches_torch_reference_and_clips():
    torch.manual_seed(0)
    c = cfg(learning_rate=1e-2, gradient_clip_threshold=0.5, weight_decay=0.1, lr_schedule="linear",
            warmup_steps_fraction=0.0, lr_final_fraction=1.0)
    p = {"w": torch.randn(5, 5), "b": torch.randn(5)}
    ref = {k: v.clone().requires_grad_(True) for k, v in p.items()}
    opt = create_optimizer(c)
    st = opt.init(p)
    topt = torch.optim.AdamW(list(ref.values()), lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    for step in range(1, 4):
        grads = {k: torch.randn_like(v) for k, v in p.items()}
        gn = math.sqrt(sum(float(g.pow(2).sum()) for g in grads.values()))
        for k in ref:
            ref[k].grad = grads[k] * (0.5 / max(gn, 0.5))
        topt.step()
        opt.update(p, grads, st, step)
    for k in p:
        assert torch.allclose(p[k], ref[k].detach(), atol=1e-5), k


def test_newton_schulz_orthogonalises():
    x = torch.randn(16, 48)
    y = oracle.newton_schulz(x, steps=8)
    sv = torch.linalg.svdvals(y)
    assert sv.max() < 1.3 and sv.min() > 0.5
    assert oracle.newton_schulz(torch.randn(3, 48, 16)).shape == (3, 48, 16)


def test_muon_update_of_a_widening_kernel_by_hand():
    """First Muon step on an [in=8, out=32] kernel, written out with plain tensor algebra (no shared helper):
    bias-corrected Nesterov momentum equals the gradient at t=1, five quintic iterations on the wide orientation,
    update scaled by sqrt(max(1, out/in)) = 2, decoupled weight decay.  The narrowing [32, 8] kernel gets scale 1."""
    torch.manual_seed(3)
    c = cfg(optimizer="muon", learning_rate=0.05, gradient_clip_threshold=0.0, weight_decay=0.1, lr_schedule="linear",
            warmup_steps_fraction=0.0, lr_final_fraction=1.0, muon_beta=0.95, muon_newton_schulz_steps=5)
    for shape, scale in (((8, 32), 2.0), ((32, 8), 1.0)):
        name = "layers.0.mlp.gate.kernel"
        w0 = torch.randn(shape)
        g = torch.randn(shape)
        p = {name: w0.clone()}
        opt = create_optimizer(c)
        st = opt.init(p)
        opt.update(p, {name: g}, st, 0)
        beta = 0.95
        mu = (1 - beta) * g
        mu_hat = beta * mu / (1 - beta ** 2) + (1 - beta) * g / (1 - beta)
        x = mu_hat if shape[0] <= shape[1] else mu_hat.t()
        x = x / (torch.sqrt((x * x).sum()) + c.adam_eps)
        for _ in range(5):
            a = x @ x.t()
            x = 3.4445 * x + (-4.7750 * a + 2.0315 * (a @ a)) @ x
        o = x if shape[0] <= shape[1] else x.t()
        lr = float(opt.schedule(0))
        want = w0 - lr * (scale * o + 0.1 * w0)
        assert torch.allclose(p[name], want, atol=1e-5), shape


@pytest.mark.parametrize("optimizer", ["adamw", "muon"])
def test_loss_decreases_on_a_fixed_batch(optimizer):
    c = cfg(optimizer=optimizer, learning_rate=3e-3 if optimizer == "adamw" else 2e-2)
    m = Transformer(c, rngs=0)
    st = trainer.create_train_state(m, c)
    b = make_batch(c)
    losses = []
    for _ in range(6):
        st, met = trainer.train_step(st, b, m, c)
        losses.append(float(met["loss"]))
    assert st.step == 6 and losses[-1] < losses[1]
    assert set(met) >= {"loss", "z_loss", "learning_rate", "grad_norm", "param_norm", "moe_expert_counts"}


def test_eval_step_and_metrics_conventions():
    c = cfg()
    m = Transformer(c, rngs=0)
    st = trainer.create_train_state(m, c)
    b = make_batch(c)
    ev = trainer.eval_step(st, b, m, c)
    before = float(trainer._l2_norm(st.params.values()))
    st, met = trainer.train_step(st, b, m, c)
    assert float(ev["eval_loss"]) == pytest.approx(float(met["loss"]), rel=1e-5)
    assert met["learning_rate"] == 0.0  # schedule value at the pre-update step
    assert float(met["param_norm"]) == pytest.approx(before, rel=1e-6)  # measured before the update


def test_grad_accumulation_equals_full_batch():
    c = cfg()
    m = Transformer(c, rngs=0)
    params = {n: p for n, p in m.named_parameters() if p.requires_grad}
    b = make_batch(c, B=4)
    loss, _ = trainer.compute_loss(None, m, c, b)
    full = torch.autograd.grad(loss, list(params.values()))
    l2, aux, acc = accumulate_gradients(lambda _p, mb: trainer.compute_loss(_p, m, c, mb), params, b, 2)
    assert float(l2) == pytest.approx(float(loss), rel=1e-5)
    for g, (n, _) in zip(full, params.items()):
        assert torch.allclose(g, acc[n], atol=1e-6), n
    c2 = cfg(gradient_accumulation_steps=2)
    st = trainer.create_train_state(m, c2)
    st, met = trainer.train_step(st, b, m, c2)
    assert float(met["loss"]) == pytest.approx(float(loss), rel=1e-5)


def test_moe_counts_bias_update_and_aux_loss():
    c = cfg(num_experts=4, num_experts_per_tok=2, moe_intermediate_size=16, n_group=2, topk_group=1,
            first_k_dense_replace=1, num_hidden_layers=3)
    m = Transformer(c, rngs=0)
    st = trainer.create_train_state(m, c)
    b = make_batch(c)
    st, met = trainer.train_step(st, b, m, c)
    counts = met["moe_expert_counts"]
    assert counts.shape == (2, 4) and int(counts[0].sum()) == 4 * 16 * 2
    st = trainer.update_expert_biases(st, counts, c)
    bias = st.params["layers.1.mlp.router.e_score_correction_bias"]
    want = c.e_score_correction_bias_update_rate * torch.sign(counts[0].float().mean() - counts[0].float())
    assert torch.allclose(bias, want)
    assert "layers.1.mlp.router.e_score_correction_bias" not in st.opt_state.mu  # never touched by the optimizer
    ca = cfg(num_experts=4, num_experts_per_tok=2, moe_intermediate_size=16, n_group=1, topk_group=1,
             first_k_dense_replace=0, router_type="softmax_topk", router_aux_loss_coef=0.1)
    ma = Transformer(ca, rngs=0)
    la, _ = trainer.compute_loss(None, ma, ca, b)
    l0, _ = trainer.compute_loss(None, ma, ca.model_copy(update={"router_aux_loss_coef": 0.0}), b)
    assert float(la) > float(l0)


def test_quantised_weight_cache_is_keyed_on_the_parameter_version():
    """The block-scaled weight copies are rebuilt when the optimizer declares the parameters changed, when a tensor
    is modified in place, and when another tensor is passed; otherwise the cached entry is returned."""
    from mintext_b200.ops import functional as F

    made = []

    def make():
        made.append(1)
        return object()

    cache = F.QuantisedWeightCache()
    w = torch.zeros(4, 4)
    a = cache.get((w,), make)
    assert cache.get((w,), make) is a and len(made) == 1
    F.bump_weight_version()
    b = cache.get((w,), make)
    assert b is not a and len(made) == 2
    w.add_(1.0)  # an in-place change moves the tensor's version counter
    c = cache.get((w,), make)
    assert c is not b and len(made) == 3
    assert cache.get((torch.zeros(4, 4),), make) is not c and len(made) == 4
