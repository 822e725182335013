"""Grouped-GEMM autotuner with an on-disk cache (reference: mintext/kernels/autotuner.py).

The reference sweeps XLA ``ragged_dot`` tile hints.  Here the tcgen05 grouped GEMM has a fixed tile, so what is
tuned is the choice that still matters at run time: candidate (tm, tk, tn) triples are timed on the machine's
actual backend (this repository's grouped kernel on a GPU, the loop oracle on CPU) for the gate/up and the down
projection, the best triple per projection is recorded together with the achieved GFLOP/s, and the result is
cached as JSON keyed by a hash of the problem (dims, dtype, device).  The cache semantics (key, file per
problem, reuse on the next call) are the reference's.
"""

from __future__ import annotations

import hashlib
import json
import time
from dataclasses import asdict, dataclass, field
from pathlib import Path

import torch

_TILE_CHOICES = (32, 64, 128, 256, 512)


@dataclass(frozen=True)
class MoETuningConfig:
    num_experts: int
    hidden_size: int
    moe_intermediate_size: int
    num_tokens: int
    dtype: str = "bfloat16"


@dataclass
class MoETuningResult:
    gate_up_tiling: tuple[int, ...]
    down_tiling: tuple[int, ...]
    backend: str = "tcgen05_grouped"
    throughput_gflops: dict = field(default_factory=dict)


def _device_kind() -> str:
    return torch.cuda.get_device_name(0) if torch.cuda.is_available() else "cpu"


def _cache_key(cfg: MoETuningConfig) -> str:
    blob = json.dumps({**asdict(cfg), "device": _device_kind()}, sort_keys=True)
    return hashlib.sha256(blob.encode()).hexdigest()[:16]


def _candidate_tilings(m: int, k: int, n: int) -> list[tuple[int, int, int]]:
    return [(tm, tk, tn) for tm in _TILE_CHOICES if tm <= m for tk in _TILE_CHOICES if tk <= k
            for tn in _TILE_CHOICES if tn <= n]


def _sample(cands, max_trials):
    if len(cands) <= max_trials:
        return cands
    step = len(cands) / max_trials
    return [cands[int(i * step)] for i in range(max_trials)]


def _time_grouped(x, w, sizes, tiling, warmup, iters) -> float:
    from mintext_b200.kernels import grouped_matmul

    for _ in range(warmup):
        grouped_matmul(x, w, sizes, tiling=tiling)
    if x.is_cuda:
        torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(iters):
        grouped_matmul(x, w, sizes, tiling=tiling)
    if x.is_cuda:
        torch.cuda.synchronize()
    return (time.perf_counter() - t0) / iters


def autotune_moe(cfg: MoETuningConfig, cache_dir: str | None = None, max_trials: int = 20, warmup_iters: int = 3,
                 bench_iters: int = 10) -> MoETuningResult:
    cache_file = None
    if cache_dir:
        Path(cache_dir).mkdir(parents=True, exist_ok=True)
        cache_file = Path(cache_dir) / f"moe_tuning_{_cache_key(cfg)}.json"
        if cache_file.exists():
            d = json.loads(cache_file.read_text())
            return MoETuningResult(tuple(d["gate_up_tiling"]), tuple(d["down_tiling"]), d["backend"],
                                   d.get("throughput_gflops", {}))
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    dt = getattr(torch, cfg.dtype) if dev == "cuda" else torch.float32
    E, D, I, M = cfg.num_experts, cfg.hidden_size, cfg.moe_intermediate_size, cfg.num_tokens
    sizes = torch.full((E,), M // E, dtype=torch.int64, device=dev)
    sizes[: M % E] += 1
    result = {}
    gflops = {}
    for name, (k, n) in (("gate_up", (D, 2 * I)), ("down", (I, D))):
        x = torch.randn(M, k, device=dev, dtype=dt)
        w = torch.randn(E, k, n, device=dev, dtype=dt)
        best, best_t = None, float("inf")
        for tiling in _sample(_candidate_tilings(M, k, n), max_trials):
            t = _time_grouped(x, w, sizes, tiling, warmup_iters, bench_iters)
            if t < best_t:
                best, best_t = tiling, t
        result[name] = best or (128, 64, 256)
        gflops[name] = 2.0 * M * k * n / best_t / 1e9 if best_t < float("inf") else 0.0
    res = MoETuningResult(tuple(result["gate_up"]), tuple(result["down"]),
                          "tcgen05_grouped" if dev == "cuda" else "loop_oracle", gflops)
    if cache_file is not None:
        cache_file.write_text(json.dumps({"gate_up_tiling": list(res.gate_up_tiling),
                                          "down_tiling": list(res.down_tiling), "backend": res.backend,
                                          "throughput_gflops": res.throughput_gflops, "config": asdict(cfg)}))
    return res
