"""Op front-ends used by the modules.

Every function takes ordinary tensors and picks the implementation:

* CUDA bf16 tensors -> the hand-written sm_100a kernels (through ``torch.autograd.Function`` wrappers defined
  here; forward and backward both run this repository's kernels);
* anything else (CPU, fp32) -> the plain-PyTorch oracle in :mod:`mintext_b200.ops.oracle`.

``set_backend("oracle")`` forces the oracle everywhere (used to cross-check the kernels on the GPU).

Weight gradients: when a parameter carries a ``main_grad`` attribute (an fp32 view into the engine's flat
gradient buffer) the wgrad GEMM accumulates straight into it with a TMA add epilogue and autograd receives
``None`` for that parameter; otherwise an ordinary gradient tensor is returned.
"""

from __future__ import annotations

import contextlib
import threading

import torch

from . import oracle
from ._ext import cuda_available, ext, status_word

_state = threading.local()


def _backend() -> str:
    return getattr(_state, "backend", "auto")


def set_backend(name: str) -> None:
    if name not in ("auto", "cuda", "oracle"):
        raise ValueError(f"backend must be auto|cuda|oracle, got {name}")
    _state.backend = name


@contextlib.contextmanager
def backend(name: str):
    prev = _backend()
    set_backend(name)
    try:
        yield
    finally:
        set_backend(prev)


def use_cuda(*tensors: torch.Tensor) -> bool:
    if _backend() == "oracle":
        return False
    t = tensors[0]
    ok = t.is_cuda and t.dtype == torch.bfloat16
    if _backend() == "cuda" and not ok:
        raise RuntimeError("backend 'cuda' needs CUDA bf16 tensors")
    return ok


# ------------------------------------------------------------------------------------------------ remat stash
class RematContext:
    """Named-activation store used by selective rematerialisation.

    During the first (no-grad) forward of a checkpointed layer, ops called with ``name=...`` deposit their
    output here when the policy saves that name; during the recompute pass the same ops fetch the stored tensor
    instead of running their kernel again, while still recording what their backward needs.
    """

    def __init__(self, save_names: frozenset[str], offload: bool = False):
        self.save_names = save_names
        self.offload = offload
        self.store: dict[str, list] = {}
        self.replay = False
        self._cursor: dict[str, int] = {}
        self._side = None

    def wants(self, name: str | None) -> bool:
        return name is not None and name in self.save_names

    def put(self, name: str, t: torch.Tensor) -> None:
        if self.offload and t.is_cuda:
            if self._side is None:
                self._side = torch.cuda.Stream()
            host = torch.empty(t.shape, dtype=t.dtype, device="cpu", pin_memory=True)
            self._side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self._side):
                host.copy_(t, non_blocking=True)
            t.record_stream(self._side)
            self.store.setdefault(name, []).append(host)
        else:
            self.store.setdefault(name, []).append(t.detach())

    def get(self, name: str, device) -> torch.Tensor | None:
        lst = self.store.get(name)
        if not lst:
            return None
        i = self._cursor.get(name, 0)
        if i >= len(lst):
            return None
        self._cursor[name] = i + 1
        t = lst[i]
        if t.device != device:
            if self._side is not None:
                torch.cuda.current_stream().wait_stream(self._side)
            t = t.to(device, non_blocking=True)
        return t

    def start_replay(self) -> None:
        self.replay = True
        self._cursor = {}


def _remat() -> RematContext | None:
    return getattr(_state, "remat", None)


@contextlib.contextmanager
def remat_scope(ctx: RematContext | None):
    prev = _remat()
    _state.remat = ctx
    try:
        yield
    finally:
        _state.remat = prev


def checkpoint_name(t: torch.Tensor, name: str) -> torch.Tensor:
    """Tag an activation with a remat name (for ops that are not linear projections)."""
    ctx = _remat()
    if ctx is not None and ctx.wants(name) and not ctx.replay:
        ctx.put(name, t)
    return t


# ------------------------------------------------------------------------------------------------ conv1d + SiLU
class _Conv1dSiluFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w):
        ctx.save_for_backward(x, w)
        return ext().conv1d_silu_fwd(x, w)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dx, dw = ext().conv1d_silu_bwd(x, w, dy.contiguous())
        return dx, dw.to(w.dtype)


def causal_conv1d_silu(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """``silu(depth-wise causal conv1d(x))``: x ``[B,S,C]``, weight ``[C,1,K]`` (mintext/modules/linear_attention.py:17-40
    followed by the activation of :123-131)."""
    C, K = weight.shape[0], weight.shape[-1]
    if (use_cuda(x) and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and C % 8 == 0 and 2 <= K <= 4
            and hasattr(ext(), "conv1d_silu_fwd")):
        return _Conv1dSiluFn.apply(x.contiguous(), weight.contiguous())
    return torch.nn.functional.silu(oracle.causal_conv1d(x, weight.to(x.dtype)))


# ------------------------------------------------------------------------------------------------ linear
def _gemm(a, b, c, a_km, b_kn, accumulate=False):
    ext().gemm(a, b, c, a_km, b_kn, accumulate, status_word(a.device))
    return c


class _LinearFn(torch.autograd.Function):
    """y[T,N] = x[T,K] @ W[K,N]  (W kept in the [in, out] layout of the parameter tree)."""

    @staticmethod
    def forward(ctx, x, w, replay_out, main_grad):
        ctx.save_for_backward(x, w)
        ctx.main_grad = main_grad
        if replay_out is not None:
            return replay_out
        y = torch.empty(x.shape[0], w.shape[1], device=x.device, dtype=torch.bfloat16)
        return _gemm(x, w, y, False, True)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy = dy.contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = torch.empty_like(x)
            _gemm(dy, w, dx, False, False)  # dy[T,N] . W[K,N]^T : W rows are K-major for this product
        if ctx.needs_input_grad[1]:
            mg = ctx.main_grad
            if mg is not None:
                _gemm(x, dy, mg.view(w.shape), True, True, accumulate=True)  # x^T dy, both MN-major
            else:
                dw = torch.empty(w.shape, device=w.device, dtype=torch.float32)
                _gemm(x, dy, dw, True, True)
                dw = dw.to(w.dtype)
        return dx, dw, None, None


def linear(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None, name: str | None = None,
           dtype: torch.dtype | None = None) -> torch.Tensor:
    """``x[..., K] @ w[K, N] (+ bias)`` computed in ``dtype`` (mintext/modules/linear.py:123-147)."""
    dtype = dtype or x.dtype
    lead = x.shape[:-1]
    K = w.shape[0]
    w2 = w.reshape(K, -1)
    rc = _remat()
    if use_cuda(x) and w2.dtype == torch.bfloat16 and K % 8 == 0 and w2.shape[1] % 8 == 0:
        x2 = x.reshape(-1, K)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        replay = rc.get(name, x.device) if (rc is not None and rc.replay and rc.wants(name)) else None
        y = _LinearFn.apply(x2, w2, replay, getattr(w, "main_grad", None))
        if rc is not None and not rc.replay and rc.wants(name):
            rc.put(name, y)
    else:
        y = x.to(dtype).reshape(-1, K) @ w2.to(dtype)
        if rc is not None and not rc.replay and rc.wants(name):
            rc.put(name, y)
    if bias is not None:
        y = y + bias.to(y.dtype)
    return y.reshape(*lead, w2.shape[1])


class _LinearFp8Fn(torch.autograd.Function):
    """``y = x @ W`` on the FP8 tensor-core path with per-tensor dynamic scales: activations e4m3 (448/amax), weights
    e5m2 (57344/amax) as in mintext/modules/linear.py:37-57.  The data gradient also runs in FP8 (output gradient
    quantised to e5m2); the weight gradient stays a bf16 GEMM accumulating in fp32."""

    @staticmethod
    def forward(ctx, x, w, main_grad):
        e, st = ext(), status_word(x.device)
        xq, _, sx = e.fp8_quantize(x, False, True, False)
        wq, wqt, sw = e.fp8_quantize(w, True, True, True)   # [K,N] for the data gradient, [N,K] for the forward
        ctx.save_for_backward(x, wq, sw)
        ctx.main_grad, ctx.wmeta = main_grad, (w.shape, w.dtype, w.device)
        return e.gemm_fp8(xq, wqt, False, True, sx, sw, st)

    @staticmethod
    def backward(ctx, dy):
        x, wq, sw = ctx.saved_tensors
        e, st = ext(), status_word(x.device)
        dy = dy.contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dyq, _, sdy = e.fp8_quantize(dy, True, True, False)
            dx = e.gemm_fp8(dyq, wq, True, True, sdy, sw, st)   # dy [T,N] . W [K,N]^T
        if ctx.needs_input_grad[1]:
            shape, wdt, dev = ctx.wmeta
            mg = ctx.main_grad
            if mg is not None:
                _gemm(x, dy, mg.view(shape), True, True, accumulate=True)
            else:
                dw = torch.empty(shape, device=dev, dtype=torch.float32)
                dw = _gemm(x, dy, dw, True, True).to(wdt)
        return dx, dw, None


def fp8_kernel_path(x: torch.Tensor, w2: torch.Tensor) -> bool:
    return (use_cuda(x) and x.dtype == torch.bfloat16 and w2.dtype == torch.bfloat16 and hasattr(ext(), "gemm_fp8")
            and w2.shape[0] % 16 == 0 and w2.shape[1] % 16 == 0)


def linear_fp8(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``x[..., K] @ w[K, N]`` through the FP8 GEMM (callers check :func:`fp8_kernel_path`)."""
    lead, K = x.shape[:-1], w.shape[0]
    x2 = x.reshape(-1, K)
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    y = _LinearFp8Fn.apply(x2, w, getattr(w, "main_grad", None))
    return y.reshape(*lead, w.shape[1])


_WEIGHT_VERSION = 0


def bump_weight_version() -> None:
    """The parameters have changed (optimizer step, checkpoint restore): quantised weight copies are stale."""
    global _WEIGHT_VERSION
    _WEIGHT_VERSION += 1


class QuantisedWeightCache:
    """Block-scaled FP8 copies of one layer's weights (both contraction orientations), kept until the parameters next
    change: with gradient accumulation and rematerialisation a weight is used many times per optimizer step but only
    changes once, so it is quantised once per step instead of once per use."""

    def __init__(self):
        self.key = None
        self.entry = None

    def get(self, tensors, make):
        key = (_WEIGHT_VERSION,) + tuple((t.data_ptr(), t._version, tuple(t.shape)) for t in tensors)
        if key != self.key:
            self.entry = make()
            self.key = key
        return self.entry


class _LinearMxfp8Fn(torch.autograd.Function):
    """``y = x @ W`` with MXFP8 operands: e4m3 elements with one power-of-two scale per 32 elements along the
    contraction, applied inside the tensor core (csrc/gemm/mxfp8_gemm.cu).  Forward and data gradient run in 8
    bits (each operand quantised along the dimension its product contracts); the weight gradient stays a bf16 GEMM
    accumulating in fp32, as on the per-tensor FP8 path (mintext/modules/linear.py:37-57 for the layer semantics)."""

    @staticmethod
    def forward(ctx, x, w, main_grad, cache):
        e, st = ext(), status_word(x.device)
        xq, xs, _, _ = e.mxfp8_quantize(x, True, False, False, False)
        # w is [K, N]: the forward contracts K (transposed copy [N, K]), the data gradient contracts N (w as stored)
        quantise = lambda: e.mxfp8_quantize(w, True, True, True, True)
        wq, ws, wqt, wst = cache.get((w,), quantise) if cache is not None else quantise()
        ctx.save_for_backward(x, wq, ws)
        ctx.main_grad, ctx.wmeta = main_grad, (w.shape, w.dtype, w.device)
        return e.gemm_mxfp8(xq, xs, wqt, wst, st)

    @staticmethod
    def backward(ctx, dy):
        x, wq, ws = ctx.saved_tensors
        e, st = ext(), status_word(x.device)
        dy = dy.contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dyq, dys, _, _ = e.mxfp8_quantize(dy, True, False, False, False)
            dx = e.gemm_mxfp8(dyq, dys, wq, ws, st)   # dy [T,N] . W [K,N]^T
        if ctx.needs_input_grad[1]:
            shape, wdt, dev = ctx.wmeta
            mg = ctx.main_grad
            if mg is not None:
                _gemm(x, dy, mg.view(shape), True, True, accumulate=True)
            else:
                dw = torch.empty(shape, device=dev, dtype=torch.float32)
                dw = _gemm(x, dy, dw, True, True).to(wdt)
        return dx, dw, None, None


class _GateUpMxfp8Fn(torch.autograd.Function):
    """``[gate | up] = x @ [Wg | Wu]`` as one block-scaled GEMM: the activation is quantised once, the concatenated
    weight is quantised once per optimizer step (``cache``), and the two weight gradients are bf16 GEMMs on the column
    halves of ``dy`` that add straight into each parameter's fp32 accumulator."""

    @staticmethod
    def forward(ctx, x, wg, wu, mg_g, mg_u, cache):
        e, st = ext(), status_word(x.device)
        xq, xs, _, _ = e.mxfp8_quantize(x, True, False, False, False)
        quantise = lambda: e.mxfp8_quantize(torch.cat([wg, wu], dim=1), True, True, True, True)
        wq, ws, wqt, wst = cache.get((wg, wu), quantise) if cache is not None else quantise()
        ctx.save_for_backward(x, wq, ws)
        ctx.grads = (mg_g, mg_u)
        ctx.wmeta = (wg.shape, wu.shape, wg.dtype, wg.device)
        return e.gemm_mxfp8(xq, xs, wqt, wst, st)

    @staticmethod
    def backward(ctx, dy):
        x, wq, ws = ctx.saved_tensors
        e, st = ext(), status_word(x.device)
        dy = dy.contiguous()
        dx = None
        if ctx.needs_input_grad[0]:
            dyq, dys, _, _ = e.mxfp8_quantize(dy, True, False, False, False)
            dx = e.gemm_mxfp8(dyq, dys, wq, ws, st)
        sg, su, wdt, dev = ctx.wmeta
        M = sg[1]
        dws = [None, None]
        for i, (need, mg, shape, cols) in enumerate(((ctx.needs_input_grad[1], ctx.grads[0], sg, slice(0, M)),
                                                     (ctx.needs_input_grad[2], ctx.grads[1], su, slice(M, M + su[1])))):
            if not need:
                continue
            if mg is not None:
                _gemm(x, dy[:, cols], mg.view(shape), True, True, accumulate=True)
            else:
                dw = torch.empty(shape, device=dev, dtype=torch.float32)
                dws[i] = _gemm(x, dy[:, cols], dw, True, True).to(wdt)
        return dx, dws[0], dws[1], None, None, None


def mxfp8_kernel_path(x: torch.Tensor, w2: torch.Tensor) -> bool:
    return (use_cuda(x) and x.dtype == torch.bfloat16 and w2.dtype == torch.bfloat16 and hasattr(ext(), "gemm_mxfp8")
            and w2.shape[0] % 128 == 0 and w2.shape[1] % 128 == 0)


def linear_mxfp8(x: torch.Tensor, w: torch.Tensor, cache: QuantisedWeightCache | None = None) -> torch.Tensor:
    """``x[..., K] @ w[K, N]`` through the block-scaled FP8 GEMM (callers check :func:`mxfp8_kernel_path`)."""
    lead, K = x.shape[:-1], w.shape[0]
    x2 = x.reshape(-1, K)
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    y = _LinearMxfp8Fn.apply(x2, w, getattr(w, "main_grad", None), cache)
    return y.reshape(*lead, w.shape[1])


def gate_up_mxfp8(x: torch.Tensor, wg: torch.Tensor, wu: torch.Tensor,
                  cache: QuantisedWeightCache | None = None) -> torch.Tensor:
    """``x[..., K] @ [wg | wu]`` -> ``[..., 2M]`` through one block-scaled FP8 GEMM."""
    lead, K = x.shape[:-1], wg.shape[0]
    x2 = x.reshape(-1, K)
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    y = _GateUpMxfp8Fn.apply(x2, wg, wu, getattr(wg, "main_grad", None), getattr(wu, "main_grad", None), cache)
    return y.reshape(*lead, wg.shape[1] + wu.shape[1])


class _LinearNTFn(torch.autograd.Function):
    """y[T,N] = x[T,K] @ W[N,K]^T (tied-embedding logits: the table is [vocab, hidden])."""

    @staticmethod
    def forward(ctx, x, w, main_grad):
        ctx.save_for_backward(x, w)
        ctx.main_grad = main_grad
        y = torch.empty(x.shape[0], w.shape[0], device=x.device, dtype=torch.bfloat16)
        return _gemm(x, w, y, False, False)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy = dy.contiguous()
        dx = torch.empty_like(x)
        _gemm(dy, w, dx, False, True)
        mg = ctx.main_grad
        if mg is not None:
            _gemm(dy, x, mg.view(w.shape), True, True, accumulate=True)
            return dx, None, None
        dw = torch.empty(w.shape, device=w.device, dtype=torch.float32)
        _gemm(dy, x, dw, True, True)
        return dx, dw.to(w.dtype), None


def linear_nt(x: torch.Tensor, w: torch.Tensor, dtype: torch.dtype | None = None) -> torch.Tensor:
    dtype = dtype or x.dtype
    lead = x.shape[:-1]
    if use_cuda(x) and w.dtype == torch.bfloat16:
        y = _LinearNTFn.apply(x.reshape(-1, x.shape[-1]).contiguous(), w, getattr(w, "main_grad", None))
    else:
        y = x.to(dtype).reshape(-1, x.shape[-1]) @ w.to(dtype).t()
    return y.reshape(*lead, w.shape[0])


# ------------------------------------------------------------------------------------------------ rmsnorm
_NORM_PARTIALS = 148 * 2


class _RMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, scale, eps, residual, main_grad):
        ctx.set_materialize_grads(False)
        ctx.main_grad = main_grad
        shape = x.shape
        dim = shape[-1]
        x2 = x.reshape(-1, dim).contiguous()
        y = torch.empty_like(x2)
        rstd = torch.empty(x2.shape[0], device=x.device, dtype=torch.float32)
        if residual is not None:
            r2 = residual.reshape(-1, dim).contiguous()
            h = torch.empty_like(x2)
            ext().rmsnorm_fwd(x2, r2, scale, y, h, rstd, eps)
        else:
            h = x2
            ext().rmsnorm_fwd(x2, None, scale, y, None, rstd, eps)
        ctx.save_for_backward(h, scale, rstd)
        ctx.has_res = residual is not None
        ctx.shape = shape
        if residual is not None:
            return y.view(shape), h.view(shape)
        return y.view(shape)

    @staticmethod
    def backward(ctx, dy, dh=None):
        h, scale, rstd = ctx.saved_tensors
        dim = h.shape[-1]
        if dy is None:  # only the summed residual stream was used downstream
            g = dh if ctx.has_res else None
            return g, None, None, g, None
        dy2 = dy.reshape(-1, dim).contiguous()
        dx = torch.empty_like(h)
        parts = torch.empty(_NORM_PARTIALS, dim, device=h.device, dtype=torch.float32)
        dres = dh.reshape(-1, dim).contiguous() if (ctx.has_res and dh is not None) else None
        mg = ctx.main_grad
        if mg is not None:
            ext().rmsnorm_bwd(h, scale, rstd, dy2, dres, dx, parts, mg, True)
            dscale = None
        else:
            dscale = torch.empty(dim, device=h.device, dtype=torch.float32)
            ext().rmsnorm_bwd(h, scale, rstd, dy2, dres, dx, parts, dscale, False)
        dxv = dx.view(ctx.shape)
        if ctx.has_res:
            return dxv, dscale, None, dxv, None
        return dxv, dscale, None, None, None


def rms_norm(x: torch.Tensor, scale: torch.Tensor, eps: float, dtype: torch.dtype | None = None) -> torch.Tensor:
    if use_cuda(x) and scale.dtype == torch.float32 and x.shape[-1] % 8 == 0:
        return _RMSNormFn.apply(x, scale, eps, None, getattr(scale, "main_grad", None))
    return oracle.rms_norm(x, scale, eps, dtype or x.dtype)


def add_rms_norm(x: torch.Tensor, residual: torch.Tensor, scale: torch.Tensor, eps: float):
    """``h = x + residual; return rms_norm(h), h`` in one pass over memory."""
    if use_cuda(x) and scale.dtype == torch.float32 and x.shape[-1] % 8 == 0:
        return _RMSNormFn.apply(x, scale, eps, residual, getattr(scale, "main_grad", None))
    h = x + residual
    return oracle.rms_norm(h, scale, eps, h.dtype), h


# ------------------------------------------------------------------------------------------------ rope
class _RopeFn(torch.autograd.Function):
    """Half-rotation RoPE, out of place.  The 16-byte vector kernel is used whenever the layout allows it (rotary
    width a multiple of 16, packed heads); the scalar in-place kernel on a copy otherwise."""

    @staticmethod
    def forward(ctx, x, cos_t, sin_t, positions, rot_dim, interleave):
        B, S, H, d = x.shape
        pos = None
        if positions is not None:
            pos = positions.reshape(-1).to(torch.int32).contiguous()
        ctx.set_materialize_grads(False)
        ctx.save_for_backward(cos_t, sin_t, pos if pos is not None else torch.empty(0))
        ctx.meta = (B, S, H, d, rot_dim, interleave, pos is not None)
        packed = x.stride(3) == 1 and x.stride(2) == d and x.stride(0) == S * x.stride(1)
        if (not interleave) and rot_dim % 16 == 0 and d % 8 == 0 and packed and x.stride(1) % 8 == 0 \
                and x.data_ptr() % 16 == 0:
            out = torch.empty(B, S, H, d, device=x.device, dtype=x.dtype)
            src = x.as_strided((B * S, H * d), (x.stride(1), 1))
            ext().rope_apply(src, out.view(B * S, H * d), cos_t, sin_t, pos, S, H, d, rot_dim, False)
            return out
        out = x.contiguous().clone()
        ext().rope(out.view(B * S, H * d), cos_t, sin_t, pos, S, H, d, rot_dim, interleave, False)
        return out

    @staticmethod
    def backward(ctx, g):
        if g is None:
            return None, None, None, None, None, None
        cos_t, sin_t, pos = ctx.saved_tensors
        B, S, H, d, rot_dim, interleave, has_pos = ctx.meta
        p = pos if has_pos else None
        g = g.contiguous()
        if (not interleave) and rot_dim % 16 == 0 and d % 8 == 0:
            dx = torch.empty_like(g)
            ext().rope_apply(g.view(B * S, H * d), dx.view(B * S, H * d), cos_t, sin_t, p, S, H, d, rot_dim, True)
            return dx, None, None, None, None, None
        dx = g.clone()
        ext().rope(dx.view(B * S, H * d), cos_t, sin_t, p, S, H, d, rot_dim, interleave, True)
        return dx, None, None, None, None, None


def rope(x: torch.Tensor, positions: torch.Tensor | None, inv_freq: torch.Tensor, attention_factor: float,
         rot_dim: int, interleave: bool, tables: tuple[torch.Tensor, torch.Tensor] | None = None,
         default_positions: bool = False) -> torch.Tensor:
    """Rotate x ``[B,S,H,d]``.  ``tables`` are cached (cos, sin) ``[max_pos, rot/2]`` used by the CUDA path;
    ``default_positions`` says positions are ``arange(S)`` for every sequence, which lets the kernel skip
    the gather."""
    if use_cuda(x) and tables is not None and tables[0].shape[0] >= x.shape[1]:
        if interleave:  # bring (2i, 2i+1) pairs to the half layout, then the ordinary rotation applies
            head = x[..., :rot_dim]
            head = head.reshape(*head.shape[:-1], -1, 2).transpose(-1, -2).reshape(head.shape)
            x = head if rot_dim == x.shape[-1] else torch.cat([head, x[..., rot_dim:]], dim=-1)
        return _RopeFn.apply(x, tables[0], tables[1], None if default_positions else positions, rot_dim, False)
    if positions is None:
        positions = torch.arange(x.shape[1], device=x.device)[None].expand(x.shape[0], -1)
    return oracle.apply_rope(x, positions, inv_freq, attention_factor, rot_dim, interleave)


# ------------------------------------------------------------------------------------------------ gated act
class _GatedActFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gate_up, act_code):
        inter = gate_up.shape[-1] // 2
        gu = gate_up.reshape(-1, 2 * inter).contiguous()
        out = torch.empty(gu.shape[0], inter, device=gu.device, dtype=gu.dtype)
        ext().gated_act_fwd(gu, out, act_code)
        ctx.save_for_backward(gu)
        ctx.act = act_code
        ctx.shape = gate_up.shape
        return out.view(*gate_up.shape[:-1], inter)

    @staticmethod
    def backward(ctx, dout):
        (gu,) = ctx.saved_tensors
        d = dout.reshape(-1, dout.shape[-1]).contiguous()
        dgu = torch.empty_like(gu)
        ext().gated_act_bwd(gu, d, dgu, ctx.act)
        return dgu.view(ctx.shape), None


def gated_act(gate_up: torch.Tensor, act: str) -> torch.Tensor:
    """``act(gate) * up`` on the column halves of a fused projection output."""
    if use_cuda(gate_up) and (gate_up.shape[-1] // 2) % 8 == 0 and act in oracle.ACT_CODES:
        return _GatedActFn.apply(gate_up, oracle.ACT_CODES[act])
    return oracle.gated_act(gate_up, act)


_GATE_MODES = {"sigmoid": 0, "silu": 1}


def _rows_view(t: torch.Tensor, dim: int) -> torch.Tensor:
    """``t`` as 2-D rows of its last dimension without copying when its leading dims collapse (a column block of a
    fused projection does); otherwise a contiguous copy."""
    try:
        return t.view(-1, dim)
    except RuntimeError:
        return t.reshape(-1, dim)


class _GateMulFn(torch.autograd.Function):
    """``x * f(gate)`` in one pass (f = sigmoid: attention output gate; f = silu: gate after the GDN head norm)."""

    @staticmethod
    def forward(ctx, x, gate, mode):
        d = x.shape[-1]
        x2, g2 = _rows_view(x, d), _rows_view(gate, d)
        out = ext().gate_mul_fwd(x2, g2, mode)
        ctx.save_for_backward(x2, g2)
        ctx.mode, ctx.shape = mode, x.shape
        return out.view(x.shape)

    @staticmethod
    def backward(ctx, dout):
        x2, g2 = ctx.saved_tensors
        dx, dg = ext().gate_mul_bwd(x2, g2, dout.reshape(x2.shape).contiguous(), ctx.mode)
        return dx.view(ctx.shape), dg.view(ctx.shape), None


def gate_mul(x: torch.Tensor, gate: torch.Tensor, kind: str) -> torch.Tensor:
    """``x * sigmoid(gate)`` or ``x * silu(gate)`` (``kind``), gate possibly a strided column block."""
    d = x.shape[-1]
    if (use_cuda(x, gate) and x.dtype == torch.bfloat16 and gate.dtype == torch.bfloat16 and x.shape == gate.shape
            and d % 8 == 0 and hasattr(ext(), "gate_mul_fwd")):
        g2 = _rows_view(gate, d)
        x2 = _rows_view(x, d)
        if g2.stride(0) % 8 == 0 and x2.stride(0) % 8 == 0 and g2.data_ptr() % 16 == 0 and x2.data_ptr() % 16 == 0:
            return _GateMulFn.apply(x, gate, _GATE_MODES[kind])
    f = torch.sigmoid(gate) if kind == "sigmoid" else torch.nn.functional.silu(gate)
    return x * f.to(x.dtype)


def _fused_gate_up(x, wg, wu, T: int, M: int) -> bool:
    import os

    return (os.environ.get("MT_FUSED_GATE_UP", "1") != "0" and hasattr(ext(), "gemm_gate_up_act") and M % 128 == 0
            and T > 128 and x.shape[1] % 8 == 0 and wg.is_contiguous() and wu.is_contiguous() and x.stride(1) == 1
            and x.stride(0) % 8 == 0)


class _GateUpActFn(torch.autograd.Function):
    """``act(x @ Wg) * (x @ Wu)``: both projections write the column halves of one ``[T, 2M]`` buffer (strided
    GEMM outputs), the activation kernel reads it once; backward mirrors this with strided dgrad / wgrad
    operands, so the gate/up pair never needs a concatenation or a fused parameter."""

    @staticmethod
    def forward(ctx, x, wg, wu, act_code, replay_buf, mg_g, mg_u):
        ctx.set_materialize_grads(False)  # the raw gate/up buffer is an auxiliary output: no zero gradient for it
        T, M = x.shape[0], wg.shape[1]
        if replay_buf is not None:
            buf = replay_buf
        else:
            buf = torch.empty(T, 2 * M, device=x.device, dtype=torch.bfloat16)
            if _fused_gate_up(x, wg, wu, T, M):
                # one CTA-pair GEMM whose accumulator holds [gate | up] for the same output columns and whose
                # epilogue also writes act(gate) * up: no separate activation kernel, no re-read of the buffer
                out = torch.empty(T, M, device=x.device, dtype=torch.bfloat16)
                ext().gemm_gate_up_act(x, wg, wu, buf, out, act_code, status_word(x.device))
                ctx.save_for_backward(x, wg, wu, buf)
                ctx.meta = (act_code, mg_g, mg_u)
                ctx.mark_non_differentiable(buf)
                return out, buf
            _gemm(x, wg, buf[:, :M], False, True)
            _gemm(x, wu, buf[:, M:], False, True)
        out = torch.empty(T, M, device=x.device, dtype=torch.bfloat16)
        ext().gated_act_fwd(buf, out, act_code)
        ctx.save_for_backward(x, wg, wu, buf)
        ctx.meta = (act_code, mg_g, mg_u)
        ctx.mark_non_differentiable(buf)
        return out, buf

    @staticmethod
    def backward(ctx, dout, _dbuf):
        x, wg, wu, buf = ctx.saved_tensors
        act_code, mg_g, mg_u = ctx.meta
        M = wg.shape[1]
        dgu = torch.empty_like(buf)
        ext().gated_act_bwd(buf, dout.contiguous(), dgu, act_code)
        dg, du = dgu[:, :M], dgu[:, M:]
        dx = torch.empty_like(x)
        _gemm(dg, wg, dx, False, False)
        _gemm(du, wu, dx, False, False, accumulate=True)
        grads = []
        for d, w, mg in ((dg, wg, mg_g), (du, wu, mg_u)):
            if mg is not None:
                _gemm(x, d, mg.view(w.shape), True, True, accumulate=True)
                grads.append(None)
            else:
                dw = torch.empty(w.shape, device=w.device, dtype=torch.float32)
                _gemm(x, d, dw, True, True)
                grads.append(dw.to(w.dtype))
        return dx, grads[0], grads[1], None, None, None, None


class _GateUpActFp8Fn(torch.autograd.Function):
    """FP8 version of the gated MLP front half: the activations are quantised once (e4m3), gate and up kernels are
    quantised together (e5m2, one scale) so that ``x @ [Wg | Wu]`` is a single FP8 GEMM writing the ``[T, 2M]``
    buffer the activation kernel reads, and the data gradient is a single FP8 GEMM over the ``2M`` columns; the
    weight gradients stay bf16 GEMMs accumulating in fp32."""

    @staticmethod
    def forward(ctx, x, wg, wu, act_code, mg_g, mg_u):
        e, st = ext(), status_word(x.device)
        T, M = x.shape[0], wg.shape[1]
        xq, _, sx = e.fp8_quantize(x, False, True, False)
        wcat = torch.cat([wg, wu], dim=1)                      # [K, 2M]
        wq, wqt, sw = e.fp8_quantize(wcat, True, True, True)   # [K, 2M] for the data gradient, [2M, K] for forward
        buf = e.gemm_fp8(xq, wqt, False, True, sx, sw, st)     # [T, 2M]
        out = torch.empty(T, M, device=x.device, dtype=torch.bfloat16)
        e.gated_act_fwd(buf, out, act_code)
        ctx.save_for_backward(x, buf, wq, sw)
        ctx.meta = (act_code, mg_g, mg_u, wg.shape, wg.dtype)
        return out

    @staticmethod
    def backward(ctx, dout):
        x, buf, wq, sw = ctx.saved_tensors
        act_code, mg_g, mg_u, wshape, wdt = ctx.meta
        e, st = ext(), status_word(x.device)
        M = wshape[1]
        dgu = torch.empty_like(buf)
        e.gated_act_bwd(buf, dout.contiguous(), dgu, act_code)
        dgq, _, sdg = e.fp8_quantize(dgu, True, True, False)
        dx = e.gemm_fp8(dgq, wq, True, True, sdg, sw, st)      # dgu [T, 2M] . [Wg | Wu][K, 2M]^T
        grads = []
        for d, mg in ((dgu[:, :M], mg_g), (dgu[:, M:], mg_u)):
            if mg is not None:
                _gemm(x, d, mg.view(wshape), True, True, accumulate=True)
                grads.append(None)
            else:
                dw = torch.empty(wshape, device=x.device, dtype=torch.float32)
                grads.append(_gemm(x, d, dw, True, True).to(wdt))
        return dx, grads[0], grads[1], None, None, None


def gate_up_act_fp8(x: torch.Tensor, wg: torch.Tensor, wu: torch.Tensor, act: str) -> torch.Tensor:
    """``act(x @ wg) * (x @ wu)`` through the FP8 GEMM (callers check :func:`fp8_kernel_path`)."""
    lead, K = x.shape[:-1], wg.shape[0]
    x2 = x.reshape(-1, K)
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    out = _GateUpActFp8Fn.apply(x2, wg, wu, oracle.ACT_CODES[act], getattr(wg, "main_grad", None),
                                getattr(wu, "main_grad", None))
    return out.reshape(*lead, wg.shape[1])


class _GatedMlpFn(torch.autograd.Function):
    """Whole gated MLP ``(act(x Wg) * (x Wu)) Wd`` as one autograd node, so that the backward can run the down
    projection's data-gradient GEMM with the activation backward in its epilogue (csrc/gemm/gated_bwd_2cta.cu): the
    gradient of the hidden activation never reaches memory.  Forward: the fused gate/up GEMM, then the down GEMM."""

    @staticmethod
    def forward(ctx, x, wg, wu, wd, act_code, mg_g, mg_u, mg_d):
        T, I = x.shape[0], wg.shape[1]
        st = status_word(x.device)
        buf = torch.empty(T, 2 * I, device=x.device, dtype=torch.bfloat16)
        h = torch.empty(T, I, device=x.device, dtype=torch.bfloat16)
        ext().gemm_gate_up_act(x, wg, wu, buf, h, act_code, st)
        y = torch.empty(T, wd.shape[1], device=x.device, dtype=torch.bfloat16)
        _gemm(h, wd, y, False, True)
        ctx.save_for_backward(x, wg, wu, wd, buf, h)
        ctx.meta = (act_code, mg_g, mg_u, mg_d)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, wg, wu, wd, buf, h = ctx.saved_tensors
        act_code, mg_g, mg_u, mg_d = ctx.meta
        I = wg.shape[1]
        dy = dy.contiguous()
        dgu = torch.empty_like(buf)
        ext().gemm_gated_bwd(dy, wd, buf, dgu, act_code, status_word(x.device))
        grads = []
        if mg_d is not None:
            _gemm(h, dy, mg_d.view(wd.shape), True, True, accumulate=True)
            dwd = None
        else:
            dwd = torch.empty(wd.shape, device=wd.device, dtype=torch.float32)
            dwd = _gemm(h, dy, dwd, True, True).to(wd.dtype)
        dg, du = dgu[:, :I], dgu[:, I:]
        dx = torch.empty_like(x)
        _gemm(dg, wg, dx, False, False)
        _gemm(du, wu, dx, False, False, accumulate=True)
        for d, w, mg in ((dg, wg, mg_g), (du, wu, mg_u)):
            if mg is not None:
                _gemm(x, d, mg.view(w.shape), True, True, accumulate=True)
                grads.append(None)
            else:
                dw = torch.empty(w.shape, device=w.device, dtype=torch.float32)
                grads.append(_gemm(x, d, dw, True, True).to(w.dtype))
        return dx, grads[0], grads[1], dwd, None, None, None, None


def gated_mlp_path(x: torch.Tensor, wg: torch.Tensor, wu: torch.Tensor, wd: torch.Tensor, act: str) -> bool:
    """The single-node gated MLP applies to bf16 CUDA tensors outside rematerialisation, with the intermediate
    width a multiple of 256 and more than one row tile."""
    import os

    if not (use_cuda(x) and _remat() is None and act in oracle.ACT_CODES and hasattr(ext(), "gemm_gated_bwd")):
        return False
    if os.environ.get("MT_FUSED_GATE_UP", "1") == "0":
        return False
    K, I = wg.shape
    rows = x.numel() // max(x.shape[-1], 1)
    return (wg.dtype == torch.bfloat16 and wu.dtype == torch.bfloat16 and wd.dtype == torch.bfloat16 and wg.dim() == 2
            and wd.dim() == 2 and wd.shape[0] == I and I % 256 == 0 and K % 8 == 0 and wd.shape[1] % 8 == 0 and rows > 128
            and wg.is_contiguous() and wu.is_contiguous() and wd.is_contiguous())


def gated_mlp(x: torch.Tensor, wg: torch.Tensor, wu: torch.Tensor, wd: torch.Tensor, act: str) -> torch.Tensor:
    """``(act(x @ wg) * (x @ wu)) @ wd`` (mintext/modules/linear.py:218-228); callers check :func:`gated_mlp_path`."""
    lead, K = x.shape[:-1], wg.shape[0]
    x2 = x.reshape(-1, K)
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    y = _GatedMlpFn.apply(x2, wg, wu, wd, oracle.ACT_CODES[act], getattr(wg, "main_grad", None),
                          getattr(wu, "main_grad", None), getattr(wd, "main_grad", None))
    return y.reshape(*lead, wd.shape[1])


def gate_up_act(x: torch.Tensor, wg: torch.Tensor, wu: torch.Tensor, act: str, dtype: torch.dtype | None = None,
                name: str = "mlp_gate_up") -> torch.Tensor:
    """Gated MLP front half, ``act(x @ wg) * (x @ wu)`` (mintext/modules/linear.py:218-225)."""
    dtype = dtype or x.dtype
    lead = x.shape[:-1]
    K, M = wg.shape
    if use_cuda(x) and wg.dtype == torch.bfloat16 and K % 8 == 0 and M % 8 == 0 and act in oracle.ACT_CODES:
        rc = _remat()
        x2 = x.reshape(-1, K)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        replay = rc.get(name, x.device) if (rc is not None and rc.replay and rc.wants(name)) else None
        out, buf = _GateUpActFn.apply(x2, wg, wu, oracle.ACT_CODES[act], replay, getattr(wg, "main_grad", None),
                                      getattr(wu, "main_grad", None))
        if rc is not None and not rc.replay and rc.wants(name):
            rc.put(name, buf)
        return out.reshape(*lead, M)
    xd = x.to(dtype)
    return oracle.activation(act)(xd @ wg.to(dtype)) * (xd @ wu.to(dtype))


# ------------------------------------------------------------------------------------------------ embedding
class _EmbeddingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, table, ids, scale, main_grad):
        ctx.main_grad = main_grad
        flat = ids.reshape(-1).contiguous()
        out = torch.empty(flat.numel(), table.shape[1], device=table.device, dtype=table.dtype)
        ext().embedding_fwd(table, flat, out, scale)
        ctx.save_for_backward(flat, table)
        ctx.scale = scale
        return out.view(*ids.shape, table.shape[1])

    @staticmethod
    def backward(ctx, dout):
        flat, table = ctx.saved_tensors
        d = dout.reshape(-1, dout.shape[-1]).contiguous()
        mg = ctx.main_grad
        if mg is not None:
            ext().embedding_bwd(d, flat, mg.view(table.shape), ctx.scale)
            return None, None, None, None
        dt = torch.zeros(table.shape, device=table.device, dtype=torch.float32)
        ext().embedding_bwd(d, flat, dt, ctx.scale)
        return dt.to(table.dtype), None, None, None


def embedding(table: torch.Tensor, ids: torch.Tensor, dtype: torch.dtype, scale: float | None = None) -> torch.Tensor:
    """Row gather, cast to ``dtype``, optional multiply by a scale rounded to ``dtype``
    (mintext/models/base.py:265-270)."""
    if table.is_cuda and table.dtype == torch.bfloat16 and dtype == torch.bfloat16 and _backend() != "oracle" \
            and table.shape[1] % 8 == 0:
        s = float(torch.tensor(scale, dtype=dtype)) if scale is not None else 1.0
        return _EmbeddingFn.apply(table, ids, s, getattr(table, "main_grad", None))
    x = table[ids].to(dtype)
    if scale is not None:
        x = x * torch.tensor(scale, dtype=dtype, device=x.device)
    return x


# ------------------------------------------------------------------------------------------------ attention
def attention(q, k, v, scale: float, causal: bool = True, window: int | None = None,
              softcap: float | None = None, mask: torch.Tensor | None = None) -> torch.Tensor:
    """Scaled-dot-product attention over ``[B,S,H,d]`` tensors with grouped-query K/V."""
    if mask is None and use_cuda(q):
        from .attention import flash_attention, flash_supported

        if flash_supported(q, k, v):
            return flash_attention(q, k, v, scale, causal, window, softcap)
    return oracle.attention(q, k, v, scale, causal, window, softcap, mask)


# ------------------------------------------------------------------------------------------------ loss
class _LinearCrossEntropyFn(torch.autograd.Function):
    """Projection to the vocabulary fused with the loss, processed in row chunks: the chunk's bf16 logits are
    produced by the GEMM, turned into gradients in place by the loss kernel, and consumed at once by the dgrad
    and wgrad GEMMs, so neither fp32 logits nor probabilities for all tokens ever exist."""

    @staticmethod
    def forward(ctx, hidden, weight, targets, weight_is_vd, ls, zw, softcap, chunk_rows, loss_scale, mg):
        N, D = hidden.shape
        V = weight.shape[0] if weight_is_vd else weight.shape[1]
        e = ext()
        st = status_word(hidden.device)
        need_grad = bool(ctx.needs_input_grad[0] or ctx.needs_input_grad[1])
        loss = torch.empty(N, device=hidden.device, dtype=torch.float32)
        zloss = torch.empty(N, device=hidden.device, dtype=torch.float32)
        dx = torch.empty_like(hidden) if need_grad else None
        dw = None
        if need_grad and mg is None:
            dw = torch.zeros(weight.shape, device=weight.device, dtype=torch.float32)
        wgrad = mg.view(weight.shape) if mg is not None else dw
        ldl = (V + 7) // 8 * 8
        logits_buf = torch.empty(min(chunk_rows, N), ldl, device=hidden.device, dtype=torch.bfloat16)
        for r0 in range(0, N, chunk_rows):
            r1 = min(N, r0 + chunk_rows)
            h = hidden[r0:r1]
            lg = logits_buf[: r1 - r0, :V]
            e.gemm(h, weight, lg, False, not weight_is_vd, False, st)
            e.cross_entropy(lg, targets[r0:r1], loss[r0:r1], zloss[r0:r1], None, ls, zw, softcap or 0.0,
                            loss_scale, need_grad)
            if need_grad:
                # dx = dlogits @ W^T(vocab-major) ; dW += (h^T dlogits) or (dlogits^T h)
                e.gemm(lg, weight, dx[r0:r1], False, weight_is_vd, False, st)
                if weight_is_vd:
                    e.gemm(lg, h, wgrad, True, True, True, st)
                else:
                    e.gemm(h, lg, wgrad, True, True, True, st)
        ctx.mark_non_differentiable(zloss)
        ctx.dx = dx
        ctx.dw = dw
        ctx.wdtype = weight.dtype
        ctx.loss_scale = loss_scale
        return loss, zloss

    @staticmethod
    def backward(ctx, dloss, dz):
        # gradients were produced in the forward for d(sum(loss) * loss_scale); the incoming dloss must be that
        # uniform scale (the trainer reduces with exactly this weighting)
        dx, dw = ctx.dx, ctx.dw
        ctx.dx = ctx.dw = None
        return dx, (dw.to(ctx.wdtype) if dw is not None else None), None, None, None, None, None, None, None, None


def linear_cross_entropy(hidden: torch.Tensor, weight: torch.Tensor, targets: torch.Tensor, *, weight_is_vd: bool,
                         label_smoothing: float = 0.0, z_loss_weight: float = 0.0, softcap: float | None = None,
                         chunk_rows: int = 4096, loss_scale: float = 1.0):
    """Per-token (loss, z_loss) of ``softmax(hidden @ W)`` against ``targets``.

    On the CUDA path the gradients w.r.t. ``hidden`` and ``W`` are computed during the forward for the objective
    ``loss_scale * sum(loss)``; the caller must reduce the returned per-token losses with that same weighting.
    """
    if use_cuda(hidden) and weight.dtype == torch.bfloat16:
        return _LinearCrossEntropyFn.apply(hidden.contiguous(), weight, targets.contiguous(), weight_is_vd,
                                           label_smoothing, z_loss_weight, softcap, chunk_rows, loss_scale,
                                           getattr(weight, "main_grad", None))
    w = weight.to(hidden.dtype)
    logits = hidden @ (w.t() if weight_is_vd else w)
    if softcap is not None:
        logits = torch.tanh(logits / softcap) * softcap
    return oracle.cross_entropy(logits, targets, label_smoothing, z_loss_weight)


__all__ = [
    "set_backend", "backend", "use_cuda", "RematContext", "remat_scope", "checkpoint_name", "linear", "linear_nt",
    "rms_norm", "add_rms_norm", "rope", "gated_act", "gate_up_act", "embedding", "attention", "linear_cross_entropy",
    "cuda_available",
]
