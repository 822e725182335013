"""Whole-model checks on the GPU: the kernel path against the oracle path, and the training engine."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _cfg(**kw):
    from mintext_b200 import MinTextConfig

    base = dict(num_hidden_layers=2, hidden_size=256, num_attention_heads=4, num_key_value_heads=2, head_dim=64,
                intermediate_size=512, vocab_size=1024, seq_length=128, per_device_batch_size=2, steps=20,
                learning_rate=1e-3, enable_tensorboard=False, enable_checkpointing=False)
    base.update(kw)
    return MinTextConfig(**base)


def _to_cuda_bf16(model):
    model.to("cuda")
    for n, p in model.named_parameters():
        if p.dim() >= 2:
            p.data = p.data.to(torch.bfloat16)
    return model


@pytest.mark.parametrize("tied", [False, True])
def test_kernel_path_matches_oracle_path(tied):
    from mintext_b200.models import Transformer
    from mintext_b200.ops import functional as F
    from mintext_b200.ops._ext import check_status
    from mintext_b200.trainer import compute_loss

    cfg = _cfg(tie_word_embeddings=tied)
    model = _to_cuda_bf16(Transformer(cfg, rngs=0))
    tok = torch.randint(0, cfg.vocab_size, (2, cfg.seq_length), device="cuda")
    batch = {"input_tokens": tok, "target_tokens": tok.roll(-1, 1)}
    params = [p for p in model.parameters() if p.requires_grad]
    loss_k, _ = compute_loss(None, model, cfg, batch)
    gk = torch.autograd.grad(loss_k, params, allow_unused=True)
    torch.cuda.synchronize()
    check_status()
    with F.backend("oracle"):
        loss_o, _ = compute_loss(None, model, cfg, batch)
        go = torch.autograd.grad(loss_o, params, allow_unused=True)
    assert abs(loss_k.item() - loss_o.item()) < 3e-2, (loss_k.item(), loss_o.item())
    bad = []
    for (n, _), a, b in zip(model.named_parameters(), gk, go):
        if a is None or b is None:
            continue
        rel = ((a.float() - b.float()).norm() / (b.float().norm() + 1e-8)).item()
        if rel > 0.1:
            bad.append((n, rel))
    assert not bad, bad


def test_engine_trains_and_matches_reference_optimizer():
    from mintext_b200.models import Transformer
    from mintext_b200.parallel.engine import TrainEngine

    cfg = _cfg()
    model = Transformer(cfg, rngs=0)
    eng = TrainEngine(model, cfg, device="cuda")
    tok = torch.randint(0, cfg.vocab_size, (4, cfg.seq_length), device="cuda")
    batch = {"input_tokens": tok, "target_tokens": tok}
    losses = [float(eng.train_step(batch, num_micro=2)["loss"]) for _ in range(8)]
    eng.check()
    assert losses[-1] < losses[0] - 0.5, losses


@pytest.mark.parametrize("policy", ["full", "save_qkv_proj", "minimal"])
def test_remat_policies_give_same_gradients(policy):
    from mintext_b200.models import Transformer
    from mintext_b200.trainer import compute_loss

    tok = torch.randint(0, 1024, (2, 128), device="cuda")
    batch = {"input_tokens": tok, "target_tokens": tok.roll(-1, 1)}
    grads = {}
    for pol in ("none", policy):
        cfg = _cfg(remat_policy=pol)
        model = _to_cuda_bf16(Transformer(cfg, rngs=0))
        params = [p for p in model.parameters() if p.requires_grad]
        loss, _ = compute_loss(None, model, cfg, batch)
        grads[pol] = (loss.item(), torch.autograd.grad(loss, params, allow_unused=True))
    assert abs(grads["none"][0] - grads[policy][0]) < 1e-3
    for a, b in zip(grads["none"][1], grads[policy][1]):
        if a is not None:
            assert torch.allclose(a.float(), b.float(), rtol=2e-2, atol=2e-3)
