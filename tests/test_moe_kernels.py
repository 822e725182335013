"""route / unroute / grouped matmul / tgmm against loop references and finite differences; autotuner cache."""

import pytest
import torch

from mintext_b200 import MinTextConfig, kernels
from mintext_b200.ops import oracle


def _setup(N=12, K=2, E=4, D=6, seed=0):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(N, D, generator=g, dtype=torch.float64)
    idx = torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(N)])
    w = torch.rand(N, K, generator=g, dtype=torch.float64)
    return x, idx, w


def test_route_shapes_contiguity_and_stability():
    x, idx, _ = _setup()
    rows, sort_idx, sizes = kernels.route(x, idx, 4)
    assert rows.shape == (24, 6) and int(sizes.sum()) == 24
    flat = idx.reshape(-1)[sort_idx]
    assert (flat[1:] >= flat[:-1]).all()
    same = flat[1:] == flat[:-1]
    assert (sort_idx[1:][same] > sort_idx[:-1][same]).all()  # stable: (token, slot) order inside an expert
    assert torch.equal(rows, x.repeat_interleave(2, 0)[sort_idx])


def test_route_unroute_roundtrip_is_weighted_sum():
    x, idx, w = _setup()
    rows, sort_idx, _ = kernels.route(x, idx, 4)
    back = kernels.unroute(rows, sort_idx, w, 2)
    assert torch.allclose(back, x * w.sum(-1, keepdim=True))


def test_route_unroute_gradients_finite_difference():
    x, idx, w = _setup(N=5, D=3)
    x.requires_grad_(True)
    w.requires_grad_(True)

    def f(x_, w_):
        rows, s, _ = kernels.route(x_, idx, 4)
        return kernels.unroute(rows * 2.0, s, w_, 2)

    assert torch.autograd.gradcheck(f, (x, w), atol=1e-6)


def test_single_and_empty_expert():
    x = torch.randn(6, 4)
    idx = torch.zeros(6, 1, dtype=torch.long)
    rows, s, sizes = kernels.route(x, idx, 3)
    assert sizes.tolist() == [6, 0, 0] and torch.equal(rows, x)


def _loop_gmm(x, w, sizes):
    out, start = [], 0
    for e, n in enumerate(sizes.tolist()):
        out.append(x[start:start + n] @ w[e])
        start += n
    return torch.cat(out)


@pytest.mark.parametrize("sizes", [[3, 3, 3, 3], [5, 0, 6, 1], [0, 0, 12, 0]])
def test_grouped_matmul_matches_loop(sizes):
    sizes = torch.tensor(sizes)
    x = torch.randn(12, 5, dtype=torch.float64)
    w = torch.randn(4, 5, 7, dtype=torch.float64)
    assert torch.allclose(kernels.grouped_matmul(x, w, sizes), _loop_gmm(x, w, sizes))
    assert torch.allclose(kernels.grouped_matmul_vjp(x, w, sizes, tiling=(128,) * 9), _loop_gmm(x, w, sizes))


def test_grouped_matmul_gradients():
    sizes = torch.tensor([2, 0, 3, 1])
    x = torch.randn(6, 4, dtype=torch.float64, requires_grad=True)
    w = torch.randn(4, 4, 3, dtype=torch.float64, requires_grad=True)
    assert torch.autograd.gradcheck(lambda a, b: kernels.grouped_matmul_vjp(a, b, sizes), (x, w), atol=1e-6)
    y = kernels.grouped_matmul_vjp(x, w, sizes)
    gx, gw = torch.autograd.grad(y.sum(), (x, w))
    y2 = _loop_gmm(x, w, sizes)
    hx, hw = torch.autograd.grad(y2.sum(), (x, w))
    assert torch.allclose(gx, hx) and torch.allclose(gw, hw)


def test_grouped_matmul_bf16():
    sizes = torch.tensor([4, 4])
    x = torch.randn(8, 16, dtype=torch.bfloat16)
    w = torch.randn(2, 16, 8, dtype=torch.bfloat16)
    out = kernels.grouped_matmul(x, w, sizes)
    assert out.dtype == torch.bfloat16
    assert torch.allclose(out.float(), _loop_gmm(x.float(), w.float(), sizes), atol=0.3, rtol=0.05)


def test_tgmm_matches_per_expert():
    sizes = torch.tensor([3, 0, 4, 1])
    lhs, rhs = torch.randn(8, 5), torch.randn(8, 6)
    out = kernels.tgmm(lhs, rhs, sizes)
    assert out.shape == (4, 5, 6)
    start = 0
    for e, n in enumerate(sizes.tolist()):
        assert torch.allclose(out[e], lhs[start:start + n].t() @ rhs[start:start + n], atol=1e-5)
        start += n
    assert float(out[1].abs().sum()) == 0


def test_moe_block_forward_backward():
    from mintext_b200.modules import MoEBlock

    c = MinTextConfig(dtype="float32", num_experts=4, num_experts_per_tok=2, moe_intermediate_size=16, n_group=2,
                      topk_group=1, hidden_size=32)
    blk = MoEBlock(c, rngs=torch.Generator().manual_seed(0))
    x = torch.randn(2, 5, 32, requires_grad=True)
    out, _ = blk(x)
    out.sum().backward()
    assert x.grad is not None and blk.experts.gate_up_proj.grad is not None
    assert blk.router.gate.kernel.grad is not None  # routing weights are differentiable


def test_autotuner_candidates_and_cache(tmp_path):
    from mintext_b200.kernels.autotuner import MoETuningConfig, MoETuningResult, _cache_key, _candidate_tilings, autotune_moe

    from mintext_b200.ops.moe import tiling_variant

    # the two tilings the tcgen05 grouped kernel exists in, mapped to its two kernel variants; one candidate on CPU
    assert _candidate_tilings(True) == [(128, 64, 256), (256, 64, 256)] and _candidate_tilings(False) == [(128, 64, 256)]
    assert [tiling_variant(t) for t in _candidate_tilings(True)] == [1, 2]
    assert tiling_variant(None) == 0 and tiling_variant(()) == 0 and tiling_variant((64, 64, 64)) == 0
    tc = MoETuningConfig(num_experts=4, hidden_size=32, moe_intermediate_size=16, num_tokens=64, dtype="float32")
    r = autotune_moe(tc, cache_dir=str(tmp_path), max_trials=2, warmup_iters=1, bench_iters=1)
    assert isinstance(r, MoETuningResult) and len(r.gate_up_tiling) == 3 and r.backend
    assert r.throughput_gflops["gate_up"] > 0 and "128x64x256" in r.throughput_gflops["gate_up_candidates_ms"]
    files = list(tmp_path.glob("*.json"))
    assert len(files) == 1
    r2 = autotune_moe(tc, cache_dir=str(tmp_path))
    assert r2.gate_up_tiling == r.gate_up_tiling
    other = MoETuningConfig(num_experts=8, hidden_size=32, moe_intermediate_size=16, num_tokens=64, dtype="float32")
    assert _cache_key(other) != _cache_key(tc)


def test_histogram_matches_bincount():
    """The sync-free expert histogram used on the training path equals ``torch.bincount(..., minlength=E)``."""
    import torch

    from mintext_b200.ops import oracle

    g = torch.Generator().manual_seed(0)
    for shape, bins in (((7, 3), 5), ((1000, 8), 128), ((1, 1), 4)):
        idx = torch.randint(0, bins, shape, generator=g)
        assert torch.equal(oracle.histogram(idx, bins), torch.bincount(idx.reshape(-1), minlength=bins))
    assert torch.equal(oracle.histogram(torch.zeros(0, dtype=torch.long), 3), torch.zeros(3, dtype=torch.long))
