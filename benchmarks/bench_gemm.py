"""Micro-benchmark: the tcgen05 bf16 GEMM against torch.matmul (cuBLAS) on the linear-layer shapes of the
Llama-3.2-1B and Llama-3-8B configs (forward, dgrad, wgrad layouts).

Timing: CUDA events, 3 warm-up runs, L2 flushed between timed runs by writing a 256 MB buffer.
Usage: python benchmarks/bench_gemm.py [--out gemm_bench.json]
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))


def _time(fn, flush, iters=10, warmup=3):
    for _ in range(warmup):
        fn()
    times = []
    for _ in range(iters):
        flush.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e))
    times.sort()
    return times[len(times) // 2]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default="")
    ap.add_argument("--tokens", type=int, default=32768)
    ap.add_argument("--only", default="", help="run only shapes whose name contains this string")
    ap.add_argument("--pair", action="store_true", help="time the CTA-pair (cta_group::2) kernel next to the 1-CTA one")
    ap.add_argument("--fp8", action="store_true", help="time the FP8 GEMM instead (ratio is against cuBLAS bf16)")
    ap.add_argument("--mxfp8", action="store_true", help="time the block-scaled FP8 GEMM instead (ratio against cuBLAS bf16)")
    args = ap.parse_args()
    from mintext_b200.ops._ext import check_status, ext, status_word

    e, st = ext(), status_word()
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    T = args.tokens
    shapes = [
        ("1b.qkv.fwd", T, 3072, 2048), ("1b.out.fwd", T, 2048, 2048), ("1b.gate_up.fwd", T, 16384, 2048),
        ("1b.down.fwd", T, 2048, 8192), ("8b.gate_up.fwd", 8192, 28672, 4096), ("8b.down.fwd", 8192, 4096, 14336),
        ("1b.lm_head.fwd", 8192, 128256, 2048),
    ]
    rows = []
    for name, M, N, K in shapes:
        if args.only and args.only not in name:
            continue
        x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
        w_kn = torch.randn(K, N, device="cuda", dtype=torch.bfloat16) * 0.02   # [in, out] storage
        dy = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
        y = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        dx = torch.empty(M, K, device="cuda", dtype=torch.bfloat16)
        dw = torch.zeros(K, N, device="cuda", dtype=torch.float32)
        dw_b = torch.empty(K, N, device="cuda", dtype=torch.bfloat16)
        flops = 2.0 * M * N * K
        cases = {
            # forward  y = x @ W          : A K-major, B stored [K,N]
            "fwd": (lambda: e.gemm(x, w_kn, y, False, True, False, st), lambda: torch.matmul(x, w_kn, out=y)),
            # dgrad    dx = dy @ W^T      : B = W as [N_out=K, contraction=N] stored K-major ([K,N] rows of length N)
            "dgrad": (lambda: e.gemm(dy, w_kn, dx, False, False, False, st), lambda: torch.matmul(dy, w_kn.t(), out=dx)),
            # wgrad    dW += x^T @ dy     : A = x stored [contraction=M, K] -> MN-major, B = dy stored [M, N]
            "wgrad": (lambda: e.gemm(x, dy, dw, True, True, True, st), lambda: torch.matmul(x.t(), dy, out=dw_b)),
        }
        if args.pair:  # CTA-pair kernel (cta_group::2) on the forward / data-gradient layouts
            cases = {
                "fwd_pair": (lambda: e.gemm_pair(x, w_kn, y, True, st), lambda: torch.matmul(x, w_kn, out=y)),
                "wgrad_auto": (lambda: e.gemm(x, dy, dw, True, True, True, st), lambda: torch.matmul(x.t(), dy, out=dw_b)),
                "dgrad_pair": (lambda: e.gemm_pair(dy, w_kn, dx, False, st), lambda: torch.matmul(dy, w_kn.t(), out=dx)),
            }
        if args.fp8:  # FP8 GEMM alone (pre-quantised operands) and the whole fp8 linear (amax + quantise + GEMM)
            xq, _, sx = e.fp8_quantize(x, False, True, False)
            _, wqt, sw = e.fp8_quantize(w_kn, True, False, True)
            cases = {
                "fp8_gemm": (lambda: e.gemm_fp8(xq, wqt, False, True, sx, sw, st), lambda: torch.matmul(x, w_kn, out=y)),
                "fp8_linear": (lambda: e.gemm_fp8(e.fp8_quantize(x, False, True, False)[0],
                                                  e.fp8_quantize(w_kn, True, False, True)[1], False, True, sx, sw, st),
                               lambda: torch.matmul(x, w_kn, out=y)),
            }
        if args.mxfp8:  # block-scaled FP8 GEMM alone (pre-quantised operands) and with both quantisations
            xq, xs, _, _ = e.mxfp8_quantize(x, True, False, False, False)
            _, _, wqt, wst = e.mxfp8_quantize(w_kn, False, False, True, True)

            def mx_linear():
                a, sa, _, _ = e.mxfp8_quantize(x, True, False, False, False)
                _, _, b, sb = e.mxfp8_quantize(w_kn, False, False, True, True)
                return e.gemm_mxfp8(a, sa, b, sb, st)

            cases = {
                "mxfp8_gemm": (lambda: e.gemm_mxfp8(xq, xs, wqt, wst, st), lambda: torch.matmul(x, w_kn, out=y)),
                "mxfp8_linear": (mx_linear, lambda: torch.matmul(x, w_kn, out=y)),
            }
        for kind, (mine, ref) in cases.items():
            t_mine = _time(mine, flush)
            t_ref = _time(ref, flush)
            check_status()
            row = {"shape": name.replace("fwd", kind), "M": M, "N": N, "K": K, "ms": round(t_mine, 4),
                   "tflops": round(flops / t_mine / 1e9, 1), "cublas_ms": round(t_ref, 4),
                   "cublas_tflops": round(flops / t_ref / 1e9, 1), "ratio": round(t_ref / t_mine, 3)}
            rows.append(row)
            print(json.dumps(row), flush=True)
        del x, w_kn, dy, y, dx, dw, dw_b
    if args.out:
        with open(args.out, "w") as f:
            json.dump(rows, f, indent=1)


if __name__ == "__main__":
    main()
