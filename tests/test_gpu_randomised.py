"""Randomised small-shape differential tests (hypothesis): kernel front-ends against the fp32 oracle on shapes the
fixed-shape tests do not enumerate - ragged tile edges, single rows, narrow and wide feature dims."""

import pytest
import torch
from hypothesis import given, settings
from hypothesis import strategies as st

pytestmark = pytest.mark.gpu
SETTINGS = dict(max_examples=20, deadline=None, derandomize=True)


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-6)).item()


@settings(**SETTINGS)
@given(m=st.integers(1, 700), n8=st.integers(1, 80), k8=st.integers(1, 80), seed=st.integers(0, 1000))
def test_linear_random_shapes(m, n8, k8, seed):
    from mintext_b200.ops import functional as F
    from mintext_b200.ops._ext import check_status

    n, k = 8 * n8, 8 * k8
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(m, k, device="cuda", generator=g).bfloat16().requires_grad_(True)
    w = (torch.randn(k, n, device="cuda", generator=g) * k ** -0.5).bfloat16().requires_grad_(True)
    y = F.linear(x, w)
    dy = torch.randn(m, n, device="cuda", generator=g).bfloat16()
    y.backward(dy)
    torch.cuda.synchronize()
    check_status()
    xf, wf = x.detach().float(), w.detach().float()
    assert _rel(y, xf @ wf) < 1e-2
    assert _rel(x.grad, dy.float() @ wf.t()) < 1e-2
    assert _rel(w.grad, xf.t() @ dy.float()) < 1e-2


@settings(**SETTINGS)
@given(rows=st.integers(1, 300), d8=st.integers(1, 512), seed=st.integers(0, 1000))
def test_rmsnorm_random_shapes(rows, d8, seed):
    from mintext_b200.ops import functional as F
    from mintext_b200.ops import oracle
    from mintext_b200.ops._ext import check_status

    d = 8 * d8
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(rows, d, device="cuda", generator=g).bfloat16().requires_grad_(True)
    scale = (1 + 0.1 * torch.randn(d, device="cuda", generator=g)).requires_grad_(True)
    y = F.rms_norm(x, scale, 1e-5)
    dy = torch.randn(rows, d, device="cuda", generator=g).bfloat16()
    y.backward(dy)
    torch.cuda.synchronize()
    check_status()
    xr, sr = x.detach().float().requires_grad_(True), scale.detach().clone().requires_grad_(True)
    with F.backend("oracle"):
        ref = oracle.rms_norm(xr, sr, 1e-5)
    ref.backward(dy.float())
    assert _rel(y, ref) < 1e-2
    assert _rel(x.grad, xr.grad) < 2e-2
    assert _rel(scale.grad, sr.grad) < 2e-2


@settings(**SETTINGS)
@given(rows=st.integers(1, 500), i8=st.integers(1, 300), act=st.sampled_from(["silu", "gelu_pytorch_tanh", "gelu", "relu"]),
       seed=st.integers(0, 1000))
def test_gated_act_random_shapes(rows, i8, act, seed):
    from mintext_b200.ops import functional as F
    from mintext_b200.ops import oracle
    from mintext_b200.ops._ext import check_status

    inter = 8 * i8
    g = torch.Generator(device="cuda").manual_seed(seed)
    gu = torch.randn(rows, 2 * inter, device="cuda", generator=g).bfloat16().requires_grad_(True)
    y = F.gated_act(gu, act)
    dy = torch.randn(rows, inter, device="cuda", generator=g).bfloat16()
    y.backward(dy)
    torch.cuda.synchronize()
    check_status()
    gr = gu.detach().float().requires_grad_(True)
    ref = oracle.gated_act(gr, act)
    ref.backward(dy.float())
    assert _rel(y, ref) < 1e-2
    assert _rel(gu.grad, gr.grad) < 2e-2
