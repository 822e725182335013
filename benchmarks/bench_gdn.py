"""Chunked Gated Delta Rule forward + backward: chunk-parallel kernels (csrc/gdn/gdn_prep.cu) + state-recurrence
kernels (csrc/gdn/gdn_scan.cu) against the plain PyTorch chunk loop, at Qwen3-Next shapes (32 value heads,
dk = dv = 128), with the time of each of the four kernels.

Usage: python benchmarks/bench_gdn.py [--B 2 --S 4096 --H 32]     (CUDA events, 2 warm-up runs, 3 timed runs)
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))


def main():
    ap = argparse.ArgumentParser()
    for k, v in (("B", 2), ("S", 4096), ("H", 32), ("d", 128)):
        ap.add_argument(f"--{k}", type=int, default=v)
    a = ap.parse_args()
    from mintext_b200.ops import oracle
    from mintext_b200.ops.gdn import chunk_gated_delta_rule_cuda

    q, k, v = (torch.randn(a.B, a.H, a.S, a.d, device="cuda", requires_grad=True) for _ in range(3))
    beta = torch.rand(a.B, a.H, a.S, device="cuda", requires_grad=True)
    g = (-torch.rand(a.B, a.H, a.S, device="cuda") * 0.5).requires_grad_(True)
    go = torch.randn(a.B, a.H, a.S, a.d, device="cuda")

    def run(fn):
        out = fn(q, k, v, beta, g)
        out.backward(go)
        for t in (q, k, v, beta, g):
            t.grad = None

    def timeit(fn, n=3):
        for _ in range(2):
            run(fn)
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        s.record()
        for _ in range(n):
            run(fn)
        e.record()
        torch.cuda.synchronize()
        return s.elapsed_time(e) / n

    t_k = timeit(chunk_gated_delta_rule_cuda)
    parts = {}
    from mintext_b200.ops._ext import ext
    from mintext_b200.ops.gdn import prep_kernel_path

    if prep_kernel_path(a.d, a.d):
        e = ext()

        def t_of(fn, n=5):
            for _ in range(2):
                fn()
            s0, e0 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            s0.record()
            for _ in range(n):
                fn()
            e0.record()
            torch.cuda.synchronize()
            return round(s0.elapsed_time(e0) / n, 3)

        with torch.no_grad():
            W, U, QG, M, KD, GL, T = e.gdn_prep_fwd(q, k, v, beta, g)
            O, S = e.gdn_scan_fwd(W, U, QG, M, KD, GL)
            dO = torch.randn_like(O)
            grads = e.gdn_scan_bwd(W, U, QG, M, KD, GL, S, dO)
            parts = {"prep_fwd_ms": t_of(lambda: e.gdn_prep_fwd(q, k, v, beta, g)),
                     "scan_fwd_ms": t_of(lambda: e.gdn_scan_fwd(W, U, QG, M, KD, GL)),
                     "scan_bwd_ms": t_of(lambda: e.gdn_scan_bwd(W, U, QG, M, KD, GL, S, dO)),
                     "prep_bwd_ms": t_of(lambda: e.gdn_prep_bwd(q, k, v, beta, g, T, *grads))}
    t_o = timeit(oracle.chunk_gated_delta_rule)
    print(json.dumps({"B": a.B, "S": a.S, "H": a.H, "d": a.d, "kernel_path_fwd_bwd_ms": round(t_k, 2),
                      "torch_chunk_loop_fwd_bwd_ms": round(t_o, 2), "speedup": round(t_o / t_k, 2), **parts}))


if __name__ == "__main__":
    main()
