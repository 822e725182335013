"""Grouped-GEMM autotuner with an on-disk cache (reference: mintext/kernels/autotuner.py).

The reference sweeps XLA ``ragged_dot`` tile hints.  The tcgen05 grouped GEMM exists in two tilings -
``(128, 64, 256)``: single-CTA tiles, and ``(256, 64, 256)``: CTA-pair tiles on two SMs (``cta_group::2``) - and
which one wins depends on the rows per expert and the projection's width, so those are the candidates on a GPU:
each is timed forward + backward (data and weight gradient) with CUDA events for the gate/up and the down
projection on expert-balanced rows, the faster one per projection is recorded together with its GFLOP/s, and the
result is cached as JSON keyed by a hash of the problem (dims, dtype, device).  ``MoEExperts`` passes the chosen
triples to the kernels (``grouped_matmul(..., tiling=...)``).  On CPU there is one implementation, so the sweep
collapses to a single candidate.  Cache semantics (key, file per problem, reuse on the next call) are the reference's.
"""

from __future__ import annotations

import hashlib
import json
import time
from dataclasses import asdict, dataclass, field
from pathlib import Path

import torch

GPU_TILINGS = ((128, 64, 256), (256, 64, 256))  # single-CTA tiles, CTA-pair tiles


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


def _candidate_tilings(on_gpu: bool) -> list[tuple[int, int, int]]:
    return list(GPU_TILINGS) if on_gpu else [GPU_TILINGS[0]]


def _time_grouped(x, w, sizes, tiling, warmup, iters) -> float:
    """Seconds per forward + backward of ``grouped_matmul`` with ``tiling`` (device-timed on a GPU)."""
    from mintext_b200.kernels import grouped_matmul

    x = x.detach().requires_grad_(True)
    w = w.detach().requires_grad_(True)

    def run():
        y = grouped_matmul(x, w, sizes, tiling=tiling)
        y.backward(y.detach())
        x.grad = w.grad = None

    for _ in range(warmup):
        run()
    if x.is_cuda:
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        for _ in range(iters):
            run()
        end.record()
        torch.cuda.synchronize()
        return start.elapsed_time(end) / 1e3 / iters
    t0 = time.perf_counter()
    for _ in range(iters):
        run()
    return (time.perf_counter() - t0) / iters


def autotune_moe(config: MoETuningConfig, cache_dir: str | None = None, max_trials: int = 20, warmup_iters: int = 3,
                 bench_iters: int = 10) -> MoETuningResult:
    cache_file = None
    if cache_dir:
        Path(cache_dir).mkdir(parents=True, exist_ok=True)
        cache_file = Path(cache_dir) / f"moe_tuning_{_cache_key(config)}.json"
        if cache_file.exists():
            d = json.loads(cache_file.read_text())
            return MoETuningResult(tuple(d["gate_up_tiling"]), tuple(d["down_tiling"]), d["backend"],
                                   d.get("throughput_gflops", {}))
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    dt = getattr(torch, config.dtype) if dev == "cuda" else torch.float32
    E, D, I, M = config.num_experts, config.hidden_size, config.moe_intermediate_size, config.num_tokens
    sizes = torch.full((E,), M // E, dtype=torch.int64, device=dev)
    sizes[: M % E] += 1
    result = {}
    gflops = {}
    for name, (k, n) in (("gate_up", (D, 2 * I)), ("down", (I, D))):
        x = torch.randn(M, k, device=dev, dtype=dt)
        w = torch.randn(E, k, n, device=dev, dtype=dt)
        best, best_t = None, float("inf")
        timings = {}
        for tiling in _candidate_tilings(dev == "cuda")[:max_trials]:
            t = _time_grouped(x, w, sizes, tiling, warmup_iters, bench_iters)
            timings["x".join(map(str, tiling))] = t
            if t < best_t:
                best, best_t = tiling, t
        result[name] = best or GPU_TILINGS[0]
        # forward + data gradient + weight gradient: three products of 2*M*k*n FLOPs
        gflops[name] = 6.0 * M * k * n / best_t / 1e9 if best_t < float("inf") else 0.0
        gflops[name + "_candidates_ms"] = {k_: round(v * 1e3, 4) for k_, v in timings.items()}
    res = MoETuningResult(tuple(result["gate_up"]), tuple(result["down"]),
                          "tcgen05_grouped" if dev == "cuda" else "loop_oracle", gflops)
    if cache_file is not None:
        cache_file.write_text(json.dumps({"gate_up_tiling": list(res.gate_up_tiling),
                                          "down_tiling": list(res.down_tiling), "backend": res.backend,
                                          "throughput_gflops": res.throughput_gflops, "config": asdict(config)}))
    return res
