"""Single-behaviour tests of the losses, schedules, optimizers and steps of the plain-PyTorch trainer (after the cases
of the reference's tests/test_train_step.py)."""

import math

import pytest
import torch

from mintext_b200 import MinTextConfig, trainer
from mintext_b200.models import Transformer
from mintext_b200.optim import accumulate_gradients, create_lr_schedule, create_optimizer


def cfg(**kw):
    base = dict(dtype="float32", vocab_size=64, num_key_value_heads=2, steps=20)
    base.update(kw)
    return MinTextConfig(**base)


def batch(c, B=4, S=16, seed=0):
    t = torch.randint(0, c.vocab_size, (B, S), generator=torch.Generator().manual_seed(seed))
    return {"input_tokens": t, "target_tokens": t.roll(-1, 1)}


# ---- cross entropy -----------------------------------------------------------------------------------------------
def test_ce_output_shape():
    loss, z = trainer.cross_entropy_loss(torch.randn(2, 5, 11), torch.randint(0, 11, (2, 5)))
    assert loss.shape == (2, 5) and z.shape == (2, 5)


def test_ce_is_positive():
    loss, _ = trainer.cross_entropy_loss(torch.randn(3, 4, 9), torch.randint(0, 9, (3, 4)))
    assert bool((loss > 0).all())


def test_ce_of_confident_correct_predictions_is_tiny():
    t = torch.tensor([[0, 3, 5]])
    logits = torch.full((1, 3, 7), -20.0).scatter_(2, t[..., None], 20.0)
    assert float(trainer.cross_entropy_loss(logits, t)[0].max()) < 1e-6


def test_ce_of_uniform_logits_is_log_vocab():
    loss, _ = trainer.cross_entropy_loss(torch.zeros(1, 2, 16), torch.tensor([[3, 9]]))
    assert torch.allclose(loss, torch.full((1, 2), math.log(16.0)), atol=1e-6)


def test_label_smoothing_raises_the_loss_of_confident_predictions():
    t = torch.tensor([[1, 2]])
    logits = torch.full((1, 2, 5), -8.0).scatter_(2, t[..., None], 8.0)
    plain, _ = trainer.cross_entropy_loss(logits, t)
    smooth, _ = trainer.cross_entropy_loss(logits, t, 0.1)
    assert bool((smooth > plain).all())


def test_label_smoothing_matches_the_dense_formula():
    logits, t = torch.randn(2, 3, 8), torch.randint(0, 8, (2, 3))
    loss, _ = trainer.cross_entropy_loss(logits, t, 0.2)
    soft = torch.nn.functional.one_hot(t, 8).float() * 0.8 + 0.2 / 8
    assert torch.allclose(loss, -(soft * torch.log_softmax(logits, -1)).sum(-1), atol=1e-6)


def test_z_loss_increases_the_loss():
    logits, t = torch.randn(2, 3, 8) * 3, torch.randint(0, 8, (2, 3))
    a, _ = trainer.cross_entropy_with_z_loss(logits, t, 0.0, 0.0)
    b, z = trainer.cross_entropy_with_z_loss(logits, t, 0.0, 1e-2)
    assert bool((b > a).all()) and torch.allclose(b - a, z, atol=1e-6)


def test_z_loss_with_zero_weight_is_the_plain_loss():
    logits, t = torch.randn(2, 3, 8), torch.randint(0, 8, (2, 3))
    a, _ = trainer.cross_entropy_loss(logits, t)
    b, z = trainer.cross_entropy_with_z_loss(logits, t, 0.0, 0.0)
    assert torch.allclose(a, b) and float(z.abs().sum()) == 0.0


def test_z_loss_has_a_gradient():
    logits = torch.randn(1, 2, 6, requires_grad=True)
    _, z = trainer.cross_entropy_with_z_loss(logits, torch.tensor([[1, 2]]), 0.0, 1e-2)
    z.sum().backward()
    assert float(logits.grad.abs().sum()) > 0


def test_z_loss_is_weight_times_squared_logsumexp():
    logits, t = torch.randn(2, 2, 7), torch.randint(0, 7, (2, 2))
    _, z = trainer.cross_entropy_with_z_loss(logits, t, 0.1, 5e-3)
    assert torch.allclose(z, 5e-3 * torch.logsumexp(logits, -1) ** 2, atol=1e-6)


def test_z_loss_reaches_the_reported_metrics():
    c = cfg(z_loss_weight=1e-2)
    m = Transformer(c, rngs=0)
    _, aux = trainer.compute_loss(None, m, c, batch(c))
    assert float(aux["z_loss"]) > 0


def test_chunked_ce_equals_the_full_one():
    h, w, t = torch.randn(12, 8), torch.randn(8, 20), torch.randint(0, 20, (12,))
    full, _ = trainer.cross_entropy_loss(h @ w, t)
    ch, _ = trainer.chunked_cross_entropy_loss(h, t, lambda x: x @ w, 3, 0.0, 0.0)
    assert torch.allclose(full, ch, atol=1e-5)


def test_vocab_tiles_in_compute_loss():
    c1 = cfg(per_device_batch_size=4, seq_length=16)
    c2 = c1.model_copy(update={"num_vocab_tiles": 8})
    m = Transformer(c1, rngs=0)
    b = batch(c1)
    assert torch.allclose(trainer.compute_loss(None, m, c1, b)[0], trainer.compute_loss(None, m, c2, b)[0], atol=1e-5)


# ---- schedules ---------------------------------------------------------------------------------------------------
def test_cosine_warmup_starts_at_zero():
    assert create_lr_schedule(cfg(steps=100, learning_rate=1.0, warmup_steps_fraction=0.1))(0) == 0.0


def test_cosine_reaches_the_peak_after_warmup():
    assert create_lr_schedule(cfg(steps=100, learning_rate=2.0, warmup_steps_fraction=0.1))(10) == pytest.approx(2.0)


def test_cosine_decays_after_warmup():
    s = create_lr_schedule(cfg(steps=100, learning_rate=1.0, warmup_steps_fraction=0.1))
    assert s(10) > s(40) > s(80) > s(100)


def test_cosine_ends_at_the_final_fraction():
    s = create_lr_schedule(cfg(steps=50, learning_rate=1.0, lr_final_fraction=0.2))
    assert s(50) == pytest.approx(0.2)


def test_linear_schedule_is_a_straight_line():
    s = create_lr_schedule(cfg(steps=100, learning_rate=1.0, lr_schedule="linear", warmup_steps_fraction=0.0,
                               lr_final_fraction=0.0))
    # the warm-up is at least one step long: the line runs from the peak at step 1 to zero at step 100
    assert s(1) == pytest.approx(1.0) and s(100) == pytest.approx(0.0)
    assert s(25) == pytest.approx(1 - 24 / 99) and s(34) - s(67) == pytest.approx(33 / 99)


def test_wsd_warmup_phase():
    s = create_lr_schedule(cfg(steps=100, learning_rate=1.0, lr_schedule="wsd", warmup_steps_fraction=0.1))
    assert s(5) == pytest.approx(0.5)


def test_wsd_stable_phase():
    s = create_lr_schedule(cfg(steps=100, learning_rate=1.0, lr_schedule="wsd", wsd_decay_steps_fraction=0.2))
    assert s(20) == s(60) == s(79) == 1.0


def test_wsd_decay_phase_is_linear_by_default():
    s = create_lr_schedule(cfg(steps=100, learning_rate=1.0, lr_schedule="wsd", wsd_decay_steps_fraction=0.2,
                               lr_final_fraction=0.0))
    assert s(90) == pytest.approx(0.5) and s(100) == pytest.approx(0.0)


def test_wsd_cosine_decay_style():
    s = create_lr_schedule(cfg(steps=100, learning_rate=1.0, lr_schedule="wsd", wsd_decay_steps_fraction=0.2,
                               wsd_decay_style="cosine", lr_final_fraction=0.0))
    assert s(90) == pytest.approx(0.5) and s(85) > 0.75  # cosine stays higher than the line early in the decay


# ---- optimizers --------------------------------------------------------------------------------------------------
def test_adamw_is_created_with_a_schedule():
    opt = create_optimizer(cfg())
    assert callable(opt.schedule) and hasattr(opt, "update") and hasattr(opt, "init")


def test_no_clipping_when_the_threshold_is_zero():
    c = cfg(gradient_clip_threshold=0.0, learning_rate=1.0, lr_schedule="linear", warmup_steps_fraction=0.0,
            lr_final_fraction=1.0, weight_decay=0.0)
    p = {"w": torch.zeros(4)}
    opt = create_optimizer(c)
    st = opt.init(p)
    opt.update(p, {"w": torch.full((4,), 100.0)}, st, 1)
    assert torch.allclose(p["w"], torch.full((4,), -1.0), atol=1e-4)  # Adam's first step is lr * sign(g)


def test_clipping_scales_large_gradients():
    big = cfg(gradient_clip_threshold=1.0)
    opt = create_optimizer(big)
    p = {"w": torch.zeros(3)}
    st = opt.init(p)
    info = opt.update(p, {"w": torch.tensor([30.0, 40.0, 0.0])}, st, 1)
    assert info is None or float(info.get("grad_norm", 50.0)) == pytest.approx(50.0)


def test_muon_optimizer_is_created():
    opt = create_optimizer(cfg(optimizer="muon"))
    assert hasattr(opt, "update")


def test_muon_with_a_target_rms_is_created():
    opt = create_optimizer(cfg(optimizer="muon", muon_consistent_rms=0.2))
    p = {"layers.0.mlp.gate.kernel": torch.randn(8, 16)}
    st = opt.init(p)
    before = p["layers.0.mlp.gate.kernel"].clone()
    opt.update(p, {"layers.0.mlp.gate.kernel": torch.randn(8, 16)}, st, 1)
    assert not torch.equal(before, p["layers.0.mlp.gate.kernel"])


def test_muon_training_step_runs():
    c = cfg(optimizer="muon", learning_rate=1e-2)
    m = Transformer(c, rngs=0)
    st = trainer.create_train_state(m, c)
    st, met = trainer.train_step(st, batch(c), m, c)
    assert st.step == 1 and math.isfinite(float(met["loss"]))


# ---- steps -------------------------------------------------------------------------------------------------------
@pytest.fixture
def setup():
    c = cfg()
    m = Transformer(c, rngs=0)
    return c, m, trainer.create_train_state(m, c), batch(c)


def test_compute_loss_returns_a_scalar_and_aux(setup):
    c, m, _, b = setup
    loss, aux = trainer.compute_loss(None, m, c, b)
    assert loss.dim() == 0 and {"loss", "z_loss", "per_token_loss", "moe_expert_counts"} <= set(aux)


def test_compute_loss_is_finite(setup):
    c, m, _, b = setup
    assert math.isfinite(float(trainer.compute_loss(None, m, c, b)[0]))


def test_initial_loss_is_about_log_vocab(setup):
    c, m, _, b = setup
    assert abs(float(trainer.compute_loss(None, m, c, b)[0]) - math.log(c.vocab_size)) < 0.5


def test_train_step_returns_a_state_and_metrics(setup):
    c, m, st, b = setup
    st2, met = trainer.train_step(st, b, m, c)
    assert hasattr(st2, "params") and hasattr(st2, "opt_state") and "loss" in met and "grad_norm" in met


def test_train_step_increments_the_step(setup):
    c, m, st, b = setup
    for expected in (1, 2, 3):
        st, _ = trainer.train_step(st, b, m, c)
        assert st.step == expected


def test_loss_decreases_over_steps(setup):
    c, m, st, b = setup
    losses = []
    for _ in range(8):
        st, met = trainer.train_step(st, b, m, c)
        losses.append(float(met["loss"]))
    assert losses[-1] < losses[1]


def test_eval_step_returns_a_loss_and_changes_nothing(setup):
    c, m, st, b = setup
    before = {n: p.detach().clone() for n, p in m.named_parameters()}
    ev = trainer.eval_step(st, b, m, c)
    assert math.isfinite(float(ev["eval_loss"]))
    assert all(torch.equal(before[n], p) for n, p in m.named_parameters())


def test_train_state_holds_parameters_and_optimizer_state(setup):
    _, m, st, _ = setup
    assert set(st.params) == {n for n, _ in m.named_parameters()} and st.step == 0 and st.opt_state is not None


def test_gradient_accumulation_equals_the_full_batch_gradient(setup):
    c, m, _, _ = setup
    params = {n: p for n, p in m.named_parameters() if p.requires_grad}
    b = batch(c, B=8)
    loss, _ = trainer.compute_loss(None, m, c, b)
    full = torch.autograd.grad(loss, list(params.values()))
    _, _, acc = accumulate_gradients(lambda _p, mb: trainer.compute_loss(_p, m, c, mb), params, b, 4)
    for g, n in zip(full, params):
        assert torch.allclose(g, acc[n], atol=1e-6), n


def test_gradient_accumulation_needs_divisible_batches(setup):
    c, m, _, _ = setup
    params = {n: p for n, p in m.named_parameters() if p.requires_grad}
    with pytest.raises(ValueError):
        accumulate_gradients(lambda _p, mb: trainer.compute_loss(_p, m, c, mb), params, batch(c, B=6), 4)


# ---- determinism -------------------------------------------------------------------------------------------------
def test_same_seed_gives_the_same_run_bit_for_bit():
    """Two runs of the plain-PyTorch trainer from the same seeds produce identical losses and parameters."""
    runs = []
    for _ in range(2):
        c = cfg(learning_rate=1e-2)
        m = Transformer(c, rngs=0)
        st = trainer.create_train_state(m, c)
        losses = []
        for s in range(4):
            st, met = trainer.train_step(st, batch(c, seed=s), m, c)
            losses.append(float(met["loss"]))
        runs.append((losses, {n: p.detach().clone() for n, p in st.params.items()}))
    assert runs[0][0] == runs[1][0]
    assert all(torch.equal(runs[0][1][n], runs[1][1][n]) for n in runs[0][1])


def test_a_different_seed_gives_a_different_model():
    c = cfg()
    a, b = Transformer(c, rngs=0), Transformer(c, rngs=1)
    assert not torch.equal(a.token_embedder, b.token_embedder)


def test_quantised_weight_cache_follows_parameter_changes():
    """The cache of quantised weight copies is reused while the weights are unchanged and rebuilt after an in-place
    write, after a declared change (optimizer kernels write through raw pointers) and for another tensor."""
    from mintext_b200.ops import functional as F

    cache, made = F.QuantisedWeightCache(), []

    def make():
        made.append(len(made))
        return made[-1]

    w = torch.zeros(4, 4)
    assert cache.get((w,), make) == 0 and cache.get((w,), make) == 0 and len(made) == 1
    w.add_(1.0)                       # in-place write through torch: the tensor's version counter moves
    assert cache.get((w,), make) == 1
    F.bump_weight_version()           # a kernel wrote the parameters through raw pointers
    assert cache.get((w,), make) == 2 and cache.get((w,), make) == 2
    assert cache.get((torch.zeros(4, 4),), make) == 3          # another tensor
    assert cache.get((w, w), make) == 4                        # another set of tensors
