"""Muon's Newton-Schulz orthogonalisation (5 iterations) on the tcgen05 GEMM kernel, per matrix shape of the
Llama-3.2-1B / Llama-3-8B layers.  FLOPs per iteration for an [r, c] matrix (r <= c): 2 r^2 c (X X^T) + 2 r^3 (A A)
+ 2 r^2 c (B X).

Usage: python benchmarks/bench_muon.py [--out file.json]      (CUDA events, 3 warm-up runs, 5 timed runs)
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
    ap.add_argument("--out", default="")
    args = ap.parse_args()
    from mintext_b200.ops import muon as muon_ops
    from mintext_b200.ops import oracle
    from mintext_b200.ops._ext import check_status

    rows = []
    for name, r, c in (("1b.qkv", 2048, 3072), ("1b.mlp", 2048, 8192), ("8b.out", 4096, 4096), ("8b.mlp", 4096, 14336)):
        x = torch.randn(1, r, c, device="cuda")
        flops = 5 * (4.0 * r * r * c + 2.0 * r ** 3)

        def timeit(fn, n=5):
            for _ in range(3):
                fn()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            s.record()
            for _ in range(n):
                fn()
            e.record()
            torch.cuda.synchronize()
            return s.elapsed_time(e) / n

        ms = timeit(lambda: muon_ops.newton_schulz(x, 5))
        ms_ref = timeit(lambda: oracle.newton_schulz(x.bfloat16(), 5))
        err = ((muon_ops.newton_schulz(x, 5) - oracle.newton_schulz(x, 5)).norm() / oracle.newton_schulz(x, 5).norm()).item()
        rows.append({"matrix": name, "rows": r, "cols": c, "ms": round(ms, 3), "tflops": round(flops / ms / 1e9, 1),
                     "torch_bf16_matmul_ms": round(ms_ref, 3), "rel_err_vs_fp32": round(err, 4)})
    check_status()
    for row in rows:
        print(json.dumps(row))
    if args.out:
        Path(args.out).write_text(json.dumps(rows, indent=1))


if __name__ == "__main__":
    main()
