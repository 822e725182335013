"""Micro-benchmark of the flash-attention kernels (forward and backward), causal, bf16.

Usage: python benchmarks/bench_attention.py [--B 8 --S 4096 --H 32 --Hkv 8 --d 64] [--iters 5] [--fwd-only]
FLOPs counted: forward 2*B*S^2*H*(d+dv)/2 (causal), backward 2.5x that.  CUDA events, 3 warm-up runs.
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
    for k, v in (("B", 8), ("S", 4096), ("H", 32), ("Hkv", 8), ("d", 64), ("dv", 0), ("iters", 5)):
        ap.add_argument(f"--{k}", type=int, default=v)
    ap.add_argument("--fwd-only", action="store_true")
    a = ap.parse_args()
    from mintext_b200.ops._ext import check_status
    from mintext_b200.ops.attention import flash_attention

    q = torch.randn(a.B, a.S, a.H, a.d, device="cuda", dtype=torch.bfloat16, requires_grad=not a.fwd_only)
    k = torch.randn(a.B, a.S, a.Hkv, a.d, device="cuda", dtype=torch.bfloat16, requires_grad=not a.fwd_only)
    dv = a.dv or a.d
    v = torch.randn(a.B, a.S, a.Hkv, dv, device="cuda", dtype=torch.bfloat16, requires_grad=not a.fwd_only)
    do = torch.randn(a.B, a.S, a.H, dv, device="cuda", dtype=torch.bfloat16)
    flops_f = 2.0 * a.B * a.S * a.S * a.H * (a.d + dv) / 2

    def timeit(fn, n):
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

    t_f = timeit(lambda: flash_attention(q, k, v, a.d ** -0.5), a.iters)
    out = {"B": a.B, "S": a.S, "H": a.H, "Hkv": a.Hkv, "d": a.d, "dv": dv, "fwd_ms": round(t_f, 3),
           "fwd_tflops": round(flops_f / t_f / 1e9, 1)}
    if not a.fwd_only:
        def fb():
            o = flash_attention(q, k, v, a.d ** -0.5)
            o.backward(do)
            q.grad = k.grad = v.grad = None

        t_fb = timeit(fb, a.iters)
        out.update({"fwd_bwd_ms": round(t_fb, 3), "bwd_ms": round(t_fb - t_f, 3),
                    "bwd_tflops": round(2.5 * flops_f / (t_fb - t_f) / 1e9, 1)})
    check_status()
    print(json.dumps(out))


if __name__ == "__main__":
    main()
