"""tcgen05 grouped GEMMs and the padded MoE pipeline against per-expert loops."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


def _check():
    from mintext_b200.ops._ext import check_status

    torch.cuda.synchronize()
    check_status()


@pytest.mark.parametrize("sizes", [[128, 128, 128, 128], [300, 0, 77, 513], [0, 0, 1000, 1], [5, 6, 7, 8]])
def test_grouped_matmul_and_grads_vs_loop(sizes):
    from mintext_b200 import kernels
    from mintext_b200.ops import oracle

    torch.manual_seed(0)
    E, K, N = len(sizes), 256, 384
    M = sum(sizes)
    gs = torch.tensor(sizes, device="cuda")
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(E, K, N, device="cuda") * 0.05).bfloat16().requires_grad_(True)
    y = kernels.grouped_matmul(x, w, gs)
    ref = oracle.grouped_matmul(x.detach().float(), w.detach().float(), gs)
    _check()
    assert _rel(y, ref) < 1e-2
    dy = torch.randn_like(y)
    y.backward(dy)
    _check()
    dx_ref = oracle.grouped_matmul(dy.float(), w.detach().float().transpose(1, 2), gs)
    dw_ref = oracle.tgmm(x.detach().float(), dy.float(), gs)
    assert _rel(x.grad, dx_ref) < 1e-2
    assert _rel(w.grad, dw_ref) < 1e-2
    t = kernels.tgmm(x.detach(), dy, gs)
    _check()
    assert _rel(t, dw_ref) < 1e-2


def test_moe_block_kernel_path_matches_oracle_path():
    from mintext_b200 import MinTextConfig
    from mintext_b200.modules import MoEBlock
    from mintext_b200.ops import functional as F

    cfg = MinTextConfig(hidden_size=256, num_experts=8, num_experts_per_tok=2, moe_intermediate_size=128, n_group=4,
                        topk_group=2, n_shared_experts=1)
    blk = MoEBlock(cfg, rngs=torch.Generator().manual_seed(0)).cuda()
    for n, p in blk.named_parameters():
        if p.dim() >= 2:
            p.data = p.data.bfloat16()
    x = torch.randn(2, 192, 256, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    out, aux = blk(x)
    params = [p for p in blk.parameters() if p.requires_grad]
    g = torch.autograd.grad(out.float().pow(2).mean(), [x] + params)
    _check()
    with F.backend("oracle"):
        out2, _ = blk(x)
        g2 = torch.autograd.grad(out2.float().pow(2).mean(), [x] + params)
    assert _rel(out, out2) < 2e-2
    for a, b in zip(g, g2):
        assert _rel(a, b) < 5e-2


def test_moe_model_trains_with_engine():
    from mintext_b200 import MinTextConfig
    from mintext_b200.models import Transformer
    from mintext_b200.parallel.engine import TrainEngine

    cfg = MinTextConfig(num_hidden_layers=2, hidden_size=256, num_attention_heads=4, num_key_value_heads=2, head_dim=64,
                        intermediate_size=512, vocab_size=1024, seq_length=128, steps=20, learning_rate=2e-3,
                        num_experts=8, num_experts_per_tok=2, moe_intermediate_size=128, n_group=1, topk_group=1,
                        first_k_dense_replace=1, n_shared_experts=0, router_type="softmax_topk",
                        router_aux_loss_coef=0.01, enable_tensorboard=False, enable_checkpointing=False)
    eng = TrainEngine(Transformer(cfg, rngs=0), cfg, device="cuda")
    tok = torch.randint(0, 1024, (4, 128), device="cuda")
    losses = []
    for _ in range(8):
        out = eng.train_step({"input_tokens": tok, "target_tokens": tok}, num_micro=1)
        losses.append(float(out["loss"]))
    eng.check()
    assert out["moe_expert_counts"].shape == (1, 8)
    assert losses[-1] < losses[1] - 0.3, losses
