"""Single-behaviour tests of the mixture-of-experts kernel API on the CPU path (route / unroute, grouped matmul with
its custom gradient, the per-expert weight-gradient product, the expert block, the autotuner's cache), after the cases
of the reference's tests/test_moe_kernels.py."""

import json

import pytest
import torch

from mintext_b200 import MinTextConfig, kernels


def _routing(N=10, K=2, E=4, D=6, seed=0, dtype=torch.float64):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(N, D, generator=g, dtype=dtype)
    idx = torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(N)])
    w = torch.rand(N, K, generator=g, dtype=dtype)
    return x, idx, w


def _loop(x, w, sizes):
    out, s = [], 0
    for e, n in enumerate(sizes.tolist()):
        out.append(x[s:s + n] @ w[e])
        s += n
    return torch.cat(out) if out else x.new_zeros(0, w.shape[-1])


# ---- route / unroute ---------------------------------------------------------------------------------------------
def test_route_output_shapes():
    x, idx, _ = _routing()
    rows, order, sizes = kernels.route(x, idx, 4)
    assert rows.shape == (20, 6) and order.shape == (20,) and sizes.shape == (4,)


def test_group_sizes_sum_to_the_number_of_assignments():
    x, idx, _ = _routing()
    assert int(kernels.route(x, idx, 4)[2].sum()) == 20


def test_group_sizes_are_the_expert_histogram():
    x, idx, _ = _routing()
    assert torch.equal(kernels.route(x, idx, 4)[2].long(), torch.bincount(idx.reshape(-1), minlength=4))


def test_rows_are_contiguous_by_expert():
    x, idx, _ = _routing()
    _, order, _ = kernels.route(x, idx, 4)
    experts = idx.reshape(-1)[order]
    assert bool((experts[1:] >= experts[:-1]).all())


def test_rows_are_copies_of_their_tokens():
    x, idx, _ = _routing()
    rows, order, _ = kernels.route(x, idx, 4)
    assert torch.equal(rows, x[order // 2])


def test_unroute_gives_one_row_per_token():
    x, idx, w = _routing()
    rows, order, _ = kernels.route(x, idx, 4)
    assert kernels.unroute(rows, order, w, 2).shape == x.shape


def test_unroute_weights_each_copy():
    x, idx, w = _routing()
    rows, order, _ = kernels.route(x, idx, 4)
    assert torch.allclose(kernels.unroute(rows, order, w, 2), x * w.sum(-1, keepdim=True))


def test_route_unroute_gradient_reaches_tokens_and_weights():
    x, idx, w = _routing()
    x.requires_grad_(True)
    w.requires_grad_(True)
    rows, order, _ = kernels.route(x, idx, 4)
    kernels.unroute(rows * 3.0, order, w, 2).sum().backward()
    assert torch.allclose(x.grad, 3.0 * w.detach().sum(-1, keepdim=True).expand_as(x))
    assert torch.allclose(w.grad, 3.0 * x.detach().sum(-1, keepdim=True).expand_as(w))


def test_route_unroute_gradient_by_finite_differences():
    x, idx, w = _routing(N=4, D=3)
    x.requires_grad_(True)
    w.requires_grad_(True)

    def f(a, b):
        rows, order, _ = kernels.route(a, idx, 4)
        return kernels.unroute(torch.tanh(rows), order, b, 2)

    assert torch.autograd.gradcheck(f, (x, w), atol=1e-6)


def test_route_with_one_expert():
    x = torch.randn(5, 3)
    rows, order, sizes = kernels.route(x, torch.zeros(5, 1, dtype=torch.long), 1)
    assert sizes.tolist() == [5] and torch.equal(rows, x) and order.tolist() == list(range(5))


def test_route_with_an_unused_expert():
    x = torch.randn(4, 3)
    idx = torch.tensor([[0], [2], [2], [0]])
    _, _, sizes = kernels.route(x, idx, 3)
    assert sizes.tolist() == [2, 0, 2]


# ---- grouped matmul ----------------------------------------------------------------------------------------------
def test_grouped_matmul_output_shape():
    out = kernels.grouped_matmul(torch.randn(9, 5), torch.randn(3, 5, 7), torch.tensor([3, 3, 3]))
    assert out.shape == (9, 7)


def test_grouped_matmul_uniform_groups():
    x, w, sizes = torch.randn(8, 4, dtype=torch.float64), torch.randn(2, 4, 3, dtype=torch.float64), torch.tensor([4, 4])
    assert torch.allclose(kernels.grouped_matmul(x, w, sizes), _loop(x, w, sizes))


def test_grouped_matmul_one_expert_is_a_plain_matmul():
    x, w = torch.randn(6, 4, dtype=torch.float64), torch.randn(1, 4, 5, dtype=torch.float64)
    assert torch.allclose(kernels.grouped_matmul(x, w, torch.tensor([6])), x @ w[0])


def test_grouped_matmul_empty_expert():
    x, w, sizes = torch.randn(5, 4, dtype=torch.float64), torch.randn(3, 4, 2, dtype=torch.float64), torch.tensor([2, 0, 3])
    assert torch.allclose(kernels.grouped_matmul(x, w, sizes), _loop(x, w, sizes))


@pytest.mark.parametrize("num_experts", [1, 2, 5, 8])
def test_grouped_matmul_expert_counts(num_experts):
    g = torch.Generator().manual_seed(num_experts)
    sizes = torch.randint(0, 5, (num_experts,), generator=g)
    x = torch.randn(int(sizes.sum()), 6, generator=g, dtype=torch.float64)
    w = torch.randn(num_experts, 6, 4, generator=g, dtype=torch.float64)
    assert torch.allclose(kernels.grouped_matmul(x, w, sizes), _loop(x, w, sizes))


def test_grouped_matmul_uneven_groups():
    sizes = torch.tensor([1, 7, 0, 2])
    x, w = torch.randn(10, 3, dtype=torch.float64), torch.randn(4, 3, 5, dtype=torch.float64)
    assert torch.allclose(kernels.grouped_matmul(x, w, sizes), _loop(x, w, sizes))


def test_grouped_matmul_bfloat16_keeps_its_dtype():
    out = kernels.grouped_matmul(torch.randn(4, 8).bfloat16(), torch.randn(2, 8, 4).bfloat16(), torch.tensor([2, 2]))
    assert out.dtype == torch.bfloat16


def test_custom_gradient_forward_equals_the_plain_product():
    sizes = torch.tensor([2, 3, 1])
    x, w = torch.randn(6, 4, dtype=torch.float64), torch.randn(3, 4, 5, dtype=torch.float64)
    assert torch.equal(kernels.grouped_matmul_vjp(x, w, sizes), kernels.grouped_matmul(x, w, sizes))


def test_custom_gradient_equals_autodiff_of_the_loop():
    sizes = torch.tensor([2, 3, 1])
    x = torch.randn(6, 4, dtype=torch.float64, requires_grad=True)
    w = torch.randn(3, 4, 5, dtype=torch.float64, requires_grad=True)
    cot = torch.randn(6, 5, dtype=torch.float64)
    gx, gw = torch.autograd.grad((kernels.grouped_matmul_vjp(x, w, sizes) * cot).sum(), (x, w))
    hx, hw = torch.autograd.grad((_loop(x, w, sizes) * cot).sum(), (x, w))
    assert torch.allclose(gx, hx) and torch.allclose(gw, hw)


def test_custom_gradient_by_finite_differences_for_the_input():
    sizes = torch.tensor([1, 2])
    x = torch.randn(3, 3, dtype=torch.float64, requires_grad=True)
    w = torch.randn(2, 3, 2, dtype=torch.float64)
    assert torch.autograd.gradcheck(lambda a: kernels.grouped_matmul_vjp(a, w, sizes), (x,), atol=1e-6)


def test_custom_gradient_by_finite_differences_for_the_weights():
    sizes = torch.tensor([1, 2])
    x = torch.randn(3, 3, dtype=torch.float64)
    w = torch.randn(2, 3, 2, dtype=torch.float64, requires_grad=True)
    assert torch.autograd.gradcheck(lambda b: kernels.grouped_matmul_vjp(x, b, sizes), (w,), atol=1e-6)


def test_nine_value_tiling_is_accepted():
    sizes = torch.tensor([2, 2])
    x, w = torch.randn(4, 4), torch.randn(2, 4, 4)
    assert torch.allclose(kernels.grouped_matmul_vjp(x, w, sizes, tiling=(128,) * 9), _loop(x, w, sizes), atol=1e-5)


def test_three_value_tiling_is_accepted():
    sizes = torch.tensor([2, 2])
    x, w = torch.randn(4, 4), torch.randn(2, 4, 4)
    assert torch.allclose(kernels.grouped_matmul_vjp(x, w, sizes, tiling=(256, 64, 256)), _loop(x, w, sizes), atol=1e-5)


def test_unused_expert_gets_a_zero_weight_gradient():
    sizes = torch.tensor([3, 0, 2])
    x = torch.randn(5, 4, dtype=torch.float64)
    w = torch.randn(3, 4, 2, dtype=torch.float64, requires_grad=True)
    kernels.grouped_matmul_vjp(x, w, sizes).sum().backward()
    assert float(w.grad[1].abs().sum()) == 0.0 and float(w.grad[0].abs().sum()) > 0


# ---- per-expert weight gradient ----------------------------------------------------------------------------------
def _loop_tgmm(lhs, rhs, sizes):
    out, s = [], 0
    for n in sizes.tolist():
        out.append(lhs[s:s + n].t() @ rhs[s:s + n])
        s += n
    return torch.stack(out)


def test_tgmm_uniform_groups():
    lhs, rhs, sizes = torch.randn(6, 3, dtype=torch.float64), torch.randn(6, 4, dtype=torch.float64), torch.tensor([2, 2, 2])
    assert torch.allclose(kernels.tgmm(lhs, rhs, sizes), _loop_tgmm(lhs, rhs, sizes))


@pytest.mark.parametrize("sizes", [[1, 5], [0, 6], [3, 0, 3], [6]])
def test_tgmm_group_sizes(sizes):
    sizes = torch.tensor(sizes)
    lhs, rhs = torch.randn(6, 3, dtype=torch.float64), torch.randn(6, 2, dtype=torch.float64)
    assert torch.allclose(kernels.tgmm(lhs, rhs, sizes), _loop_tgmm(lhs, rhs, sizes))


def test_tgmm_empty_group_is_zero():
    out = kernels.tgmm(torch.randn(4, 3), torch.randn(4, 2), torch.tensor([4, 0]))
    assert float(out[1].abs().sum()) == 0.0


def test_tgmm_bfloat16():
    out = kernels.tgmm(torch.randn(4, 8).bfloat16(), torch.randn(4, 8).bfloat16(), torch.tensor([2, 2]))
    assert out.shape == (2, 8, 8)


# ---- the expert block and a model with it ------------------------------------------------------------------------
def _moe_cfg(**kw):
    base = dict(dtype="float32", num_experts=4, num_experts_per_tok=2, moe_intermediate_size=16, n_group=2, topk_group=1,
                hidden_size=32, vocab_size=64, num_key_value_heads=2, first_k_dense_replace=0)
    base.update(kw)
    return MinTextConfig(**base)


def test_moe_block_forward_shape_and_aux():
    from mintext_b200.modules import MoEBlock

    blk = MoEBlock(_moe_cfg(), rngs=torch.Generator().manual_seed(0))
    out, aux = blk(torch.randn(2, 5, 32))
    assert out.shape == (2, 5, 32) and aux["topk_indices"].shape == (10, 2) and aux["scores"].shape == (10, 4)


def test_moe_block_backward_reaches_every_parameter_group():
    from mintext_b200.modules import MoEBlock

    blk = MoEBlock(_moe_cfg(n_shared_experts=1), rngs=torch.Generator().manual_seed(0))
    x = torch.randn(2, 5, 32, requires_grad=True)
    blk(x)[0].sum().backward()
    assert x.grad is not None
    for p in (blk.experts.gate_up_proj, blk.experts.down_proj, blk.router.gate.kernel, blk.shared_expert.gate.kernel):
        assert p.grad is not None and float(p.grad.abs().sum()) > 0


def test_moe_block_selection_bias_has_no_gradient():
    from mintext_b200.modules import MoEBlock

    blk = MoEBlock(_moe_cfg(), rngs=torch.Generator().manual_seed(0))
    blk(torch.randn(1, 4, 32))[0].sum().backward()
    assert blk.router.e_score_correction_bias.grad is None and not blk.router.e_score_correction_bias.requires_grad


def test_transformer_with_expert_layers_runs():
    from mintext_b200.models import Transformer

    c = _moe_cfg(num_hidden_layers=2)
    out, aux = Transformer(c, rngs=0)(torch.randint(0, 64, (2, 8)))
    assert out.shape == (2, 8, 64) and len([a for a in aux if a is not None]) == 2


def test_training_step_with_expert_layers():
    from mintext_b200 import trainer
    from mintext_b200.models import Transformer

    c = _moe_cfg(num_hidden_layers=2, steps=10)
    m = Transformer(c, rngs=0)
    st = trainer.create_train_state(m, c)
    t = torch.randint(0, 64, (4, 8), generator=torch.Generator().manual_seed(0))
    st, met = trainer.train_step(st, {"input_tokens": t, "target_tokens": t}, m, c)
    assert met["moe_expert_counts"].shape == (2, 4) and int(met["moe_expert_counts"].sum()) == 2 * 4 * 8 * 2


# ---- autotuner ---------------------------------------------------------------------------------------------------
def _tuning_cfg(**kw):
    from mintext_b200.kernels.autotuner import MoETuningConfig

    base = dict(num_experts=4, hidden_size=32, moe_intermediate_size=16, num_tokens=64, dtype="float32")
    base.update(kw)
    return MoETuningConfig(**base)


def test_autotuner_candidates_are_the_kernels_that_exist():
    from mintext_b200.kernels.autotuner import _candidate_tilings

    assert _candidate_tilings(True) == [(128, 64, 256), (256, 64, 256)] and len(_candidate_tilings(False)) == 1


def test_autotuner_writes_one_cache_file(tmp_path):
    from mintext_b200.kernels.autotuner import autotune_moe

    autotune_moe(_tuning_cfg(), cache_dir=str(tmp_path), max_trials=1, warmup_iters=1, bench_iters=1)
    files = list(tmp_path.glob("*.json"))
    assert len(files) == 1 and "gate_up_tiling" in json.loads(files[0].read_text())


def test_autotuner_reads_its_cache(tmp_path):
    from mintext_b200.kernels.autotuner import autotune_moe

    a = autotune_moe(_tuning_cfg(), cache_dir=str(tmp_path), max_trials=1, warmup_iters=1, bench_iters=1)
    stamp = next(tmp_path.glob("*.json")).stat().st_mtime_ns
    b = autotune_moe(_tuning_cfg(), cache_dir=str(tmp_path))
    assert (a.gate_up_tiling, a.down_tiling) == (b.gate_up_tiling, b.down_tiling)
    assert next(tmp_path.glob("*.json")).stat().st_mtime_ns == stamp


def test_autotuner_cache_key_depends_on_the_problem():
    from mintext_b200.kernels.autotuner import _cache_key

    keys = {_cache_key(_tuning_cfg()), _cache_key(_tuning_cfg(num_experts=8)), _cache_key(_tuning_cfg(hidden_size=64)),
            _cache_key(_tuning_cfg(num_tokens=128)), _cache_key(_tuning_cfg(dtype="bfloat16"))}
    assert len(keys) == 5


def test_autotuner_result_fields(tmp_path):
    from mintext_b200.kernels.autotuner import MoETuningResult, autotune_moe

    r = autotune_moe(_tuning_cfg(), cache_dir=str(tmp_path), max_trials=1, warmup_iters=1, bench_iters=1)
    assert isinstance(r, MoETuningResult) and len(r.gate_up_tiling) == 3 and len(r.down_tiling) == 3 and r.backend
    assert r.throughput_gflops["gate_up"] > 0 and r.throughput_gflops["down"] > 0
