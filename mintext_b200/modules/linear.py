"""Linear projections and the gated MLP (reference: mintext/modules/linear.py).

Kernels keep the reference's parameter-tree shapes: ``in_shape + out_shape`` with the input dims first, e.g.
``[D, H, dh]`` for a head-expanding projection and ``[H, dh, D]`` for the contracting output projection.  The
GEMM kernel reads ``[in, out]`` weights directly (MN-major B operand), so no transposed copy is kept.
"""

from __future__ import annotations

import math
from typing import Sequence

import torch
from torch import nn

from mintext_b200.ops import functional as F
from mintext_b200.ops import oracle


def _as_tuple(v) -> tuple[int, ...]:
    return tuple(v) if isinstance(v, (tuple, list)) else (int(v),)


_INIT_DEVICE: torch.device | None = None


class init_on_device:
    """While active, parameter initialisers draw their values on ``device`` instead of the host.

    Building a multi-billion-parameter model on the host costs minutes of single-threaded sampling and, with one
    process per GPU, eight host copies of the weights; on the GPU the same tensors appear in milliseconds and only
    the slices a rank keeps stay allocated.  Device streams are seeded from the model's host generator (one draw per
    tensor), so a given seed still names one set of weights - though not the set the host path draws."""

    def __init__(self, device):
        self.device = torch.device(device) if device is not None else None

    def __enter__(self):
        global _INIT_DEVICE
        self._prev = _INIT_DEVICE
        _INIT_DEVICE = self.device if (self.device is not None and self.device.type == "cuda") else None
        return self

    def __exit__(self, *exc):
        global _INIT_DEVICE
        _INIT_DEVICE = self._prev


def _device_generator(generator: torch.Generator | None) -> torch.Generator:
    seed = int(torch.randint(0, 2 ** 31 - 1, (1,), generator=generator)) if generator is not None else 0
    return torch.Generator(device=_INIT_DEVICE).manual_seed(seed)


def normal_init(shape: Sequence[int], std: float, generator: torch.Generator | None,
                dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """``N(0, std^2)`` values (embedding tables, convolution taps)."""
    if _INIT_DEVICE is not None:
        t = torch.empty(tuple(shape), dtype=torch.float32, device=_INIT_DEVICE)
        t.normal_(0.0, std, generator=_device_generator(generator))
        return t.to(dtype)
    return (torch.randn(tuple(shape), generator=generator) * std).to(dtype)


def truncated_normal_init(shape: Sequence[int], fan_in: int, generator: torch.Generator | None,
                          dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """Standard normal truncated to [-2, 2], times ``1/sqrt(fan_in)`` with no variance correction
    (mintext/modules/linear.py:18-30)."""
    if _INIT_DEVICE is not None:
        t = torch.empty(tuple(shape), dtype=torch.float32, device=_INIT_DEVICE)
        nn.init.trunc_normal_(t, mean=0.0, std=1.0, a=-2.0, b=2.0, generator=_device_generator(generator))
        return t.mul_(1.0 / math.sqrt(max(fan_in, 1))).to(dtype)
    t = torch.empty(tuple(shape), dtype=torch.float32)
    nn.init.trunc_normal_(t, mean=0.0, std=1.0, a=-2.0, b=2.0, generator=generator)
    return (t / math.sqrt(max(fan_in, 1))).to(dtype)


def variance_scaling_init(scale: float = 1.0):
    """Initialiser factory with the reference's calling convention (mintext/modules/linear.py:18-30):
    ``init(generator, shape, dtype, in_axis, out_axis)`` draws a standard normal truncated to [-2, 2] and multiplies
    it by ``scale / sqrt(fan_in)``, where ``fan_in`` is the product of the dims that are not output axes.
    ``in_axis`` is accepted for signature parity; the fan-in follows from ``out_axis`` as in the reference."""

    def init(generator, shape, dtype=torch.float32, in_axis=0, out_axis=-1):
        outs = out_axis if isinstance(out_axis, (tuple, list)) else (out_axis,)
        fan_out = 1
        for a in outs:
            fan_out *= int(shape[a])
        fan_in = max(math.prod(int(d) for d in shape) // max(fan_out, 1), 1)
        t = truncated_normal_init(shape, fan_in, generator, torch.float32)
        return (t * float(scale)).to(dtype)

    return init


def fp8_matmul_reference(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """Per-tensor dynamically scaled fp8 product: activations to e4m3 with ``448/amax``, weights to e5m2 with
    ``57344/amax``, fp32 accumulation, rescale (mintext/modules/linear.py:37-57)."""
    xa = x.float().abs().max().clamp_min(1e-12)
    wa = w.float().abs().max().clamp_min(1e-12)
    sx, sw = 448.0 / xa, 57344.0 / wa
    xq = (x.float() * sx).to(torch.float8_e4m3fn).float()
    wq = (w.float() * sw).to(torch.float8_e5m2).float()
    return ((xq @ wq) / (sx * sw)).to(out_dtype)


def mxfp8_matmul_reference(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """Block-scaled fp8 product ``x[T,K] @ w[K,N]``: both operands to e4m3 with one power-of-two scale per 32
    elements along K (the smallest that brings the block within +-448), fp32 accumulation.  Torch statement of
    what csrc/gemm/mxfp8_gemm.cu computes; used where the kernel path is unavailable."""
    def qdq(t: torch.Tensor) -> torch.Tensor:  # blocks along the last dim
        r, k = t.shape
        pad = (-k) % 32
        tf = torch.nn.functional.pad(t.float(), (0, pad)).view(r, -1, 32)
        amax = tf.abs().amax(-1, keepdim=True)
        e = torch.ceil(torch.log2(amax.clamp_min(2.0 ** -120) / 448.0)).clamp(-127, 127)
        scale = torch.exp2(e)
        q = (tf / scale).clamp(-448, 448).to(torch.float8_e4m3fn).float() * scale
        return q.view(r, -1)[:, :k]

    return (qdq(x) @ qdq(w.t()).t()).to(out_dtype)


class Linear(nn.Module):
    """``in_features`` / ``out_features`` may be ints or tuples (head-shaped kernels)."""

    def __init__(self, in_features, out_features, dtype: torch.dtype = torch.float32,
                 weight_dtype: torch.dtype = torch.float32, kernel_axes: tuple = (), use_bias: bool = False,
                 kernel_init_fn=None, use_fp8: bool = False, *, rngs: torch.Generator | None = None,
                 name: str | None = None, fp8_recipe: str = "per_tensor"):
        super().__init__()
        self.in_shape = _as_tuple(in_features)
        self.out_shape = _as_tuple(out_features)
        self.dtype = dtype
        self.use_fp8 = use_fp8
        self.fp8_recipe = str(fp8_recipe)
        self.remat_name = name
        fan_in = math.prod(self.in_shape)
        shape = self.in_shape + self.out_shape
        init = kernel_init_fn or truncated_normal_init
        self.kernel = nn.Parameter(init(shape, fan_in, rngs, weight_dtype))
        self.kernel.logical_axes = tuple(kernel_axes)
        if use_bias:
            self.bias = nn.Parameter(torch.zeros(self.out_shape, dtype=weight_dtype))
            self.bias.logical_axes = tuple(kernel_axes[len(self.in_shape):])
        else:
            self.bias = None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        n_in = len(self.in_shape)
        lead = x.shape[: x.dim() - n_in]
        fan_in = math.prod(self.in_shape)
        x2 = x.reshape(*lead, fan_in)
        w2 = self.kernel.reshape(fan_in, -1) if self.kernel.dim() != 2 else self.kernel
        if self.use_fp8 and self.kernel.dim() == 2 and self.fp8_recipe == "mx_block":
            if F.mxfp8_kernel_path(x2, w2):
                if not hasattr(self, "_mx_cache"):
                    self._mx_cache = F.QuantisedWeightCache()
                y = F.linear_mxfp8(x2, w2, self._mx_cache)
            else:
                y = mxfp8_matmul_reference(x2.reshape(-1, fan_in), w2, self.dtype).reshape(*lead, -1)
            if self.bias is not None:
                y = y + self.bias.to(y.dtype).reshape(-1)
        elif self.use_fp8 and self.kernel.dim() == 2 and F.fp8_kernel_path(x2, w2):
            y = F.linear_fp8(x2, w2)
            if self.bias is not None:
                y = y + self.bias.to(y.dtype).reshape(-1)
        elif self.use_fp8 and self.kernel.dim() == 2:
            y = fp8_matmul_reference(x2.reshape(-1, fan_in), w2, self.dtype).reshape(*lead, -1)
            if self.bias is not None:
                y = y + self.bias.to(y.dtype).reshape(-1)
        else:
            if w2 is not self.kernel and hasattr(self.kernel, "main_grad"):
                w2.main_grad = self.kernel.main_grad
            y = F.linear(x2, w2, None if self.bias is None else self.bias.reshape(-1), name=self.remat_name,
                         dtype=self.dtype)
        return y.reshape(*lead, *self.out_shape)


class MLP(nn.Module):
    """Gated feed-forward ``down(act(gate(x)) * up(x))`` (mintext/modules/linear.py:174-228).

    ``gate`` and ``up`` are separate parameters (``[D, M]`` each) as in the reference tree.
    """

    def __init__(self, config, *, rngs: torch.Generator | None = None, mesh=None, intermediate_size: int | None = None):
        super().__init__()
        D = config.hidden_size
        M = intermediate_size or config.intermediate_size
        dt, wdt = config.torch_dtype, config.torch_weight_dtype
        self.act_name = config.hidden_activation
        fp8 = bool(config.use_fp8)
        rec = str(getattr(config, "fp8_recipe", "per_tensor"))
        # block-scaled copies of [gate | up] and down, re-made when the optimizer has changed the weights
        self._mx_gate_up, self._mx_down = F.QuantisedWeightCache(), F.QuantisedWeightCache()
        self.gate = Linear(D, M, dt, wdt, ("embed", "mlp"), use_fp8=fp8, rngs=rngs, name="mlp_gate_proj", fp8_recipe=rec)
        self.up = Linear(D, M, dt, wdt, ("embed", "mlp"), use_fp8=fp8, rngs=rngs, name="mlp_up", fp8_recipe=rec)
        self.down = Linear(M, D, dt, wdt, ("mlp", "embed"), use_fp8=fp8, rngs=rngs, name="mlp_down", fp8_recipe=rec)
        from mintext_b200.parallel.tp import current_tp

        self.tp = current_tp() if (current_tp() is not None and current_tp().size > 1) else None
        if self.tp is not None:
            lo, hi = self.tp.shard(M, "intermediate_size")
            for lin, dim in ((self.gate, 1), (self.up, 1), (self.down, 0)):
                full = lin.kernel.data
                axes = lin.kernel.logical_axes
                lin.kernel = nn.Parameter((full[:, lo:hi] if dim == 1 else full[lo:hi]).clone().contiguous())
                lin.kernel.logical_axes = axes
                lin.kernel.tensor_parallel = True
                lin.kernel.shard_spec = (dim, self.tp.rank, self.tp.size)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.tp is not None:
            from mintext_b200.parallel import tp as tpm

            lead, D = x.shape[:-1], x.shape[-1]
            x2 = x.reshape(-1, D)
            if self.gate.use_fp8 and self.gate.fp8_recipe == "mx_block" and self.act_name in oracle.ACT_CODES \
                    and F.mxfp8_kernel_path(x2, self.gate.kernel) and F.mxfp8_kernel_path(x2, self.down.kernel):
                # block-scaled FP8 on the rank's column / row slices: the gathered tokens are quantised once for
                # gate|up; the collectives around the two GEMMs are the group's all-gather and reduce-scatter
                xg = tpm.all_gather_tokens(x2, self.tp)
                gu = F.gate_up_mxfp8(xg, self.gate.kernel, self.up.kernel, self._mx_gate_up)
                h = F.gated_act(gu, self.act_name)
                return tpm.reduce_scatter_tokens(F.linear_mxfp8(h, self.down.kernel, self._mx_down), self.tp).view(*lead, D)
            _, (g, u) = tpm.column_linear(x.reshape(-1, D), [self.gate.kernel, self.up.kernel], self.tp, self.gate.dtype)
            h = F.gated_act(torch.cat([g, u], dim=-1), self.act_name)
            return tpm.row_linear(h, self.down.kernel, self.tp, self.gate.dtype).view(*lead, D)
        if self.gate.use_fp8 and self.gate.fp8_recipe == "mx_block":
            x2 = x.reshape(-1, x.shape[-1])
            if self.act_name in oracle.ACT_CODES and F.mxfp8_kernel_path(x2, self.gate.kernel):
                # one block-scaled GEMM for gate|up (the activation is quantised once), then the gated-act kernel
                gu = F.gate_up_mxfp8(x, self.gate.kernel, self.up.kernel, self._mx_gate_up)
                h = F.gated_act(gu, self.act_name)
                if self.down.bias is None and F.mxfp8_kernel_path(h.reshape(-1, h.shape[-1]), self.down.kernel):
                    return F.linear_mxfp8(h, self.down.kernel, self._mx_down)
            else:
                h = oracle.activation(self.act_name)(self.gate(x)) * self.up(x)
        elif self.gate.use_fp8 and self.act_name in oracle.ACT_CODES and \
                F.fp8_kernel_path(x.reshape(-1, x.shape[-1]), self.gate.kernel):
            h = F.gate_up_act_fp8(x, self.gate.kernel, self.up.kernel, self.act_name)
        elif self.gate.use_fp8:
            h = oracle.activation(self.act_name)(self.gate(x)) * self.up(x)
        else:
            if self.down.bias is None and F.gated_mlp_path(x, self.gate.kernel, self.up.kernel, self.down.kernel,
                                                           self.act_name):
                return F.gated_mlp(x, self.gate.kernel, self.up.kernel, self.down.kernel, self.act_name)
            h = F.gate_up_act(x, self.gate.kernel, self.up.kernel, self.act_name, dtype=self.gate.dtype)
        return self.down(h)


ACT2FN = {name: oracle.activation(name) for name in ("silu", "gelu", "gelu_pytorch_tanh", "relu")}
