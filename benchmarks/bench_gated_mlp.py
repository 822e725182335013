"""Gated MLP forward + backward: the single-node path (gate|up GEMM with the activation in its epilogue; down-projection
data-gradient GEMM with the activation backward in its epilogue) against separate GEMMs + activation kernels.

    python benchmarks/bench_gated_mlp.py [--T 32768 --D 2048 --I 8192] [--iters 5]

FLOPs counted: 3 GEMM passes x 2 x T x D x 3I.  CUDA events, 3 warm-ups; the working set (> 1 GB) exceeds L2.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))


def main():
    ap = argparse.ArgumentParser()
    for k, v in (("T", 32768), ("D", 2048), ("I", 8192), ("iters", 5)):
        ap.add_argument(f"--{k}", type=int, default=v)
    ap.add_argument("--only", choices=("fused", "separate"), default=None)
    a = ap.parse_args()
    from mintext_b200.ops import functional as F
    from mintext_b200.ops._ext import check_status

    x = torch.randn(a.T, a.D, device="cuda").bfloat16().requires_grad_(True)
    wg = (torch.randn(a.D, a.I, device="cuda") * a.D ** -0.5).bfloat16().requires_grad_(True)
    wu = (torch.randn(a.D, a.I, device="cuda") * a.D ** -0.5).bfloat16().requires_grad_(True)
    wd = (torch.randn(a.I, a.D, device="cuda") * a.I ** -0.5).bfloat16().requires_grad_(True)
    for w in (wg, wu, wd):  # accumulate weight gradients in fp32 as the engine does
        w.main_grad = torch.zeros(w.shape, device="cuda", dtype=torch.float32)
    dy = torch.randn(a.T, a.D, device="cuda").bfloat16()
    flops = 3 * 2.0 * a.T * a.D * 3 * a.I

    def run(fused: bool) -> float:
        os.environ["MT_FUSED_GATE_UP"] = "1" if fused else "0"

        def step():
            if fused:
                y = F.gated_mlp(x, wg, wu, wd, "silu")
            else:
                y = F.linear(F.gate_up_act(x, wg, wu, "silu"), wd)
            y.backward(dy)
            x.grad = None

        for _ in range(3):
            step()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        s.record()
        for _ in range(a.iters):
            step()
        e.record()
        torch.cuda.synchronize()
        check_status()
        return s.elapsed_time(e) / a.iters

    out = {"T": a.T, "D": a.D, "I": a.I}
    for name, fused in (("fused", True), ("separate", False)):
        if a.only and a.only != name:
            continue
        ms = run(fused)
        out[name + "_ms"] = round(ms, 3)
        out[name + "_tflops"] = round(flops / ms / 1e9, 1)
    print(json.dumps(out))


if __name__ == "__main__":
    main()
