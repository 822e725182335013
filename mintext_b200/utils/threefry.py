"""Counter-based synthetic token stream: Threefry-2x32 (20 rounds) and the key-splitting / ``randint``
constructions the reference's synthetic batches come from (mintext/train.py:55-66,165-176 draws
``jax.random.randint(key, (B, S), 0, V)`` from a key that is split once per step).

Because every element is a pure function of ``(key, flat index)``, a rank can produce exactly its own rows of the
global batch, on the device, with no host generator state and no host-to-device copy; and a resumed run lands on
the same stream by splitting the key ``start_step`` times.  The construction follows JAX's published algorithm in
its default ("partitionable") form: the bits of element ``i`` are ``y0 ^ y1`` of ``threefry2x32(key, (hi32(i),
lo32(i)))``; ``split`` takes both words; ``randint`` combines two 32-bit draws to remove modulo bias.  JAX is not
available in this build to compare against, so the cipher is pinned by the Random123 known-answer vectors and the
rest by this module's own CPU / GPU cross-checks.
"""

from __future__ import annotations

import torch

_M = 0xFFFFFFFF
_ROT = ((13, 15, 26, 6), (17, 29, 16, 24))
_PARITY = 0x1BD11BDA


def _rotl(x, r):
    return ((x << r) | (x >> (32 - r))) & _M


def threefry2x32(k0, k1, x0, x1):
    """One Threefry-2x32-20 block.  Works on Python ints and on int64 tensors holding 32-bit values."""
    ks = (k0 & _M, k1 & _M, (k0 ^ k1 ^ _PARITY) & _M)
    x0 = (x0 + ks[0]) & _M
    x1 = (x1 + ks[1]) & _M
    for g in range(5):
        for r in _ROT[g % 2]:
            x0 = (x0 + x1) & _M
            x1 = _rotl(x1, r) ^ x0
        x0 = (x0 + ks[(g + 1) % 3]) & _M
        x1 = (x1 + ks[(g + 2) % 3] + g + 1) & _M
    return x0, x1


def key(seed: int) -> tuple[int, int]:
    """Key of an integer seed: (high word, low word)."""
    seed = int(seed)
    return (seed >> 32) & _M, seed & _M


def split(k: tuple[int, int], num: int = 2) -> list[tuple[int, int]]:
    """``num`` independent keys: key ``i`` is the cipher block of counter ``i``."""
    return [threefry2x32(k[0], k[1], 0, i) for i in range(num)]


def random_bits(k: tuple[int, int], start: int, count: int, device="cpu") -> torch.Tensor:
    """32 random bits (as int64) for flat indices ``start .. start + count``."""
    idx = torch.arange(start, start + count, dtype=torch.int64, device=device)
    y0, y1 = threefry2x32(k[0], k[1], idx >> 32, idx & _M)
    return y0 ^ y1


def randint_rows(k: tuple[int, int], row_lo: int, rows: int, cols: int, maxval: int, device="cpu",
                 use_kernel: bool | None = None) -> torch.Tensor:
    """Rows ``row_lo .. row_lo + rows`` of ``randint(key, (any, cols), 0, maxval)`` as int64 ``[rows, cols]``."""
    span = int(maxval)
    if not 0 < span <= _M:
        raise ValueError(f"maxval must be in 1 .. 2**32 - 1, got {maxval}")
    k1, k2 = split(k)
    device = torch.device(device)
    if use_kernel is None:
        use_kernel = device.type == "cuda"
    if use_kernel:
        from mintext_b200.ops._ext import ext

        out = torch.empty(rows, cols, dtype=torch.int64, device=device)
        ext().threefry_randint(out, k1[0], k1[1], k2[0], k2[1], row_lo * cols, span)
        return out
    hi = random_bits(k1, row_lo * cols, rows * cols, device)
    lo = random_bits(k2, row_lo * cols, rows * cols, device)
    mult = (1 << 16) % span
    mult = (mult * mult) % span
    off = (((hi % span) * mult) & _M) + (lo % span)   # 32-bit wrap-around of the product, as unsigned hardware does
    return ((off & _M) % span).view(rows, cols)


def randint(k: tuple[int, int], shape: tuple[int, int], maxval: int, device="cpu") -> torch.Tensor:
    return randint_rows(k, 0, shape[0], shape[1], maxval, device)
