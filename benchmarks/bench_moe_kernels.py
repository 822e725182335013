"""MoE kernel micro-benchmark (the reference's benchmarks/benchmark_moe_kernels.py shapes): grouped GEMM forward,
backward (data + weight gradient) and forward+backward, in GFLOP/s, tcgen05 grouped kernel vs a per-expert loop of
torch.matmul (cuBLAS).

Usage: python benchmarks/bench_moe_kernels.py [--shapes small,dsv3,llama_moe] [--out file.json]
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

SHAPES = {  # name: (experts, hidden, intermediate, top_k, tokens)
    "tiny": (4, 128, 256, 2, 256),
    "small": (8, 512, 1024, 2, 1024),
    "medium": (16, 1024, 2048, 4, 2048),
    "qwen3_30b": (128, 2048, 768, 8, 16384),
    "dsv3": (256, 7168, 2048, 8, 4096),
    "llama_moe": (8, 4096, 14336, 2, 4096),
}


def _time(fn, iters=5, warmup=3):
    for _ in range(warmup):
        fn()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) / iters


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--shapes", default="small,medium,qwen3_30b,dsv3,llama_moe")
    ap.add_argument("--out", default="")
    args = ap.parse_args()
    from mintext_b200 import kernels
    from mintext_b200.ops._ext import check_status

    rows = []
    for name in args.shapes.split(","):
        E, D, I, K, T = SHAPES[name]
        M = T * K
        sizes = torch.full((E,), M // E, device="cuda", dtype=torch.int64)
        sizes[: M % E] += 1
        x = torch.randn(M, D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
        w = (torch.randn(E, D, 2 * I, device="cuda") * 0.02).bfloat16().requires_grad_(True)
        dy = torch.randn(M, 2 * I, device="cuda", dtype=torch.bfloat16)
        flops = 2.0 * M * D * 2 * I
        starts = torch.cumsum(sizes, 0).tolist()

        def loop():
            out, s0 = [], 0
            for e, s1 in enumerate(starts):
                out.append(x.detach()[s0:s1] @ w.detach()[e])
                s0 = s1
            return out

        def fwd():
            return kernels.grouped_matmul(x, w, sizes)

        def fwd_bwd():
            y = kernels.grouped_matmul(x, w, sizes)
            y.backward(dy)
            x.grad = w.grad = None

        t_f, t_fb, t_loop = _time(fwd), _time(fwd_bwd), _time(loop)
        check_status()
        row = {"shape": name, "E": E, "D": D, "I": I, "rows": M, "fwd_ms": round(t_f, 4),
               "fwd_tflops": round(flops / t_f / 1e9, 1), "fwd_bwd_ms": round(t_fb, 4),
               "fwd_bwd_tflops": round(3 * flops / t_fb / 1e9, 1), "cublas_loop_fwd_ms": round(t_loop, 4),
               "cublas_loop_fwd_tflops": round(flops / t_loop / 1e9, 1)}
        rows.append(row)
        print(json.dumps(row), flush=True)
    if args.out:
        Path(args.out).write_text(json.dumps(rows, indent=1))


if __name__ == "__main__":
    main()
