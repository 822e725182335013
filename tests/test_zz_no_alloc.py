"""The allocation-free RMSNorm backward entry point, called through its exported C symbol.

Some hosts of this library may not allocate device memory where they call it (inside a stream capture, in a
serving loop with a fixed memory plan, or when another runtime owns the allocator), so ``mt_rmsnorm_bwd_noalloc``
keeps its scratch inside the library.  This test calls the symbol with ctypes, twice in a row (the second call
reuses the scratch the first one left behind), and compares both results with the ordinary entry point.
"""

import ctypes
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from mintext_b200.ops._ext import ext

    ext()  # make sure the shared object is built and loaded
    path = Path(__file__).resolve().parents[1] / "mintext_b200" / "_mt_C.so"
    lib = ctypes.CDLL(str(path))
    fn = lib.mt_rmsnorm_bwd_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 7 + [ctypes.c_int64, ctypes.c_int, ctypes.c_int, ctypes.c_void_p,
                                           ctypes.c_char_p, ctypes.c_size_t]
    return fn


def _reference(x, w, rstd, dy, dres):
    from mintext_b200.ops._ext import ext

    dx = torch.empty_like(x)
    parts = torch.empty(64, x.shape[1], device="cuda")
    dw = torch.zeros(x.shape[1], device="cuda")
    ext().rmsnorm_bwd(x, w, rstd, dy, dres, dx, parts, dw, False)
    return dx, dw


def _call(fn, x, w, rstd, dy, dres, accumulate=0, dw=None, dx=None):
    dx = torch.empty_like(x) if dx is None else dx
    dw = torch.zeros(x.shape[1], device="cuda") if dw is None else dw
    err = ctypes.create_string_buffer(256)
    stream = torch.cuda.current_stream().cuda_stream
    rc = fn(x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dy.data_ptr(), dres.data_ptr() if dres is not None else None,
            dx.data_ptr(), dw.data_ptr(), x.shape[0], x.shape[1], accumulate, stream, err, 256)
    return rc, err.value.decode(), dx, dw


def test_no_alloc_entry_point_matches_ordinary_one_twice():
    fn = _lib()
    torch.manual_seed(0)
    for call, (rows, dim) in enumerate([(777, 2048), (1500, 4096)]):
        x = torch.randn(rows, dim, device="cuda", dtype=torch.bfloat16)
        dy = torch.randn(rows, dim, device="cuda", dtype=torch.bfloat16)
        dres = torch.randn(rows, dim, device="cuda", dtype=torch.bfloat16) if call == 1 else None
        w = (1 + 0.1 * torch.randn(dim, device="cuda")).float()
        rstd = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-5)
        # outputs exist before the call, so anything that appears on the device during it was allocated by it:
        # neither torch's caching allocator nor the driver (free memory of the device) may move
        dx = torch.empty_like(x)
        dw = torch.zeros(dim, device="cuda")
        if call == 0:
            assert _call(fn, x, w, rstd, dy, dres, dw=dw, dx=dx)[0] == 0  # first call on the device: address look-up
        torch.cuda.synchronize()
        allocated, reserved, free = torch.cuda.memory_allocated(), torch.cuda.memory_reserved(), torch.cuda.mem_get_info()[0]
        rc, msg, dx, dw = _call(fn, x, w, rstd, dy, dres, dw=dw, dx=dx)
        torch.cuda.synchronize()
        assert rc == 0, msg
        assert torch.cuda.memory_allocated() == allocated and torch.cuda.memory_reserved() == reserved
        assert torch.cuda.mem_get_info()[0] >= free, "device memory shrank during an allocation-free call"
        ref_dx, ref_dw = _reference(x, w, rstd, dy, dres)
        torch.cuda.synchronize()
        assert torch.equal(dx, ref_dx)
        assert torch.allclose(dw, ref_dw, rtol=1e-2, atol=1e-2)  # same tolerance as the other RMSNorm tests
        rel = ((dw - ref_dw).norm() / ref_dw.norm()).item()
        assert rel < 1e-2, rel


def test_no_alloc_entry_point_accumulates_and_rejects_oversize():
    fn = _lib()
    x = torch.randn(64, 1024, device="cuda", dtype=torch.bfloat16)
    dy = torch.randn_like(x)
    w = torch.ones(1024, device="cuda")
    rstd = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-5)
    _, _, _, once = _call(fn, x, w, rstd, dy, None)
    acc = once.clone()
    rc, msg, _, twice = _call(fn, x, w, rstd, dy, None, accumulate=1, dw=acc)
    torch.cuda.synchronize()
    assert rc == 0 and torch.allclose(twice, 2 * once, rtol=1e-5, atol=1e-5)
    big = torch.zeros(8, 16384, device="cuda", dtype=torch.bfloat16)
    rc, msg, _, _ = _call(fn, big, torch.ones(16384, device="cuda"), torch.ones(8, device="cuda"), big, None)
    assert rc != 0 and "exceeds the built-in scratch limit" in msg
    rc, msg, _, _ = _call(fn, x[:, :1020].contiguous(), w[:1020].contiguous(), rstd, dy[:, :1020].contiguous(), None)
    assert rc != 0 and "multiple of 8" in msg


def test_no_alloc_entry_point_with_no_rows_writes_the_empty_sum():
    fn = _lib()
    dim = 512
    x = torch.empty(0, dim, device="cuda", dtype=torch.bfloat16)
    w = torch.ones(dim, device="cuda")
    rstd = torch.empty(0, device="cuda")
    stale = torch.full((dim,), 7.0, device="cuda")
    rc, msg, _, dw = _call(fn, x, w, rstd, x, None, accumulate=0, dw=stale.clone())
    torch.cuda.synchronize()
    assert rc == 0, msg
    assert torch.count_nonzero(dw).item() == 0            # a sum over zero rows
    rc, msg, _, dw = _call(fn, x, w, rstd, x, None, accumulate=1, dw=stale.clone())
    torch.cuda.synchronize()
    assert rc == 0 and torch.equal(dw, stale)             # accumulating nothing leaves dw alone
