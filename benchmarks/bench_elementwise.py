"""Bandwidth-bound kernels at Llama-3.2-1B shapes (32768 tokens): achieved GB/s against the measured HBM copy rate.

RMSNorm forward / backward (with residual), RoPE forward / backward, gated activation forward / backward, fused
linear + cross-entropy (one 4096-row chunk sequence over the 128256-entry vocabulary), causal conv1d + SiLU.
Bytes counted are the algorithmic minimum (each operand read once, each result written once).

Usage: python benchmarks/bench_elementwise.py [--tokens 32768] [--only rmsnorm] [--out file.json]
Timing: CUDA events, 3 warm-up runs, 10 timed runs; tensors (64 MB to 1 GB) exceed or rival the 126 MB L2.
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))


def _time(fn, iters=10, warmup=3):
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
    ap.add_argument("--tokens", type=int, default=32768)
    ap.add_argument("--only", default="")
    ap.add_argument("--out", default="")
    args = ap.parse_args()
    from mintext_b200.ops import functional as F
    from mintext_b200.ops._ext import check_status

    peak = 6522.7
    pk = Path(__file__).resolve().parents[1] / "MEASURED_PEAKS.json"
    if pk.exists():
        peak = float(json.loads(pk.read_text()).get("hbm_gbs", peak))
    T, D, H, Hkv, dh, Fm, V = args.tokens, 2048, 32, 8, 64, 8192, 128256
    dev = "cuda"
    rows = []

    def add(name, fn, nbytes):
        if args.only and args.only not in name:
            return
        ms = _time(fn)
        gbs = nbytes / ms / 1e6
        rows.append({"kernel": name, "ms": round(ms, 4), "GB": round(nbytes / 1e9, 3), "GBps": round(gbs, 1),
                     "frac_of_measured_hbm": round(gbs / peak, 3)})

    x = torch.randn(T, D, device=dev).bfloat16().requires_grad_(True)
    res = torch.randn(T, D, device=dev).bfloat16().requires_grad_(True)
    scale = torch.ones(D, device=dev, requires_grad=True)
    with torch.no_grad():
        add("rmsnorm_fwd (+residual)", lambda: F.add_rms_norm(x, res, scale, 1e-5), 4 * T * D * 2)
    y, h = F.add_rms_norm(x, res, scale, 1e-5)
    gy, gh = torch.randn_like(y), torch.randn_like(h)
    add("rmsnorm fwd+bwd (+residual)", lambda: torch.autograd.grad(F.add_rms_norm(x, res, scale, 1e-5), (x, res, scale), (gy, gh)),
        (4 + 4) * T * D * 2)

    B, S = T // 4096, 4096
    q = torch.randn(B, S, H, dh, device=dev).bfloat16().requires_grad_(True)
    inv = 1.0 / (500000.0 ** (torch.arange(0, dh, 2, device=dev).float() / dh))
    ang = torch.arange(S, device=dev).float()[:, None] * inv[None]
    tables = (ang.cos().contiguous(), ang.sin().contiguous())
    with torch.no_grad():
        add("rope_fwd (32 heads)", lambda: F.rope(q, None, inv, 1.0, dh, False, tables, True), 2 * q.numel() * 2)
    gq = torch.randn_like(q)
    add("rope fwd+bwd", lambda: torch.autograd.grad(F.rope(q, None, inv, 1.0, dh, False, tables, True), q, gq),
        4 * q.numel() * 2)

    gu = torch.randn(T, 2 * Fm, device=dev).bfloat16().requires_grad_(True)
    with torch.no_grad():
        add("swiglu_fwd", lambda: F.gated_act(gu, "silu"), 3 * T * Fm * 2)
    go = torch.randn(T, Fm, device=dev).bfloat16()
    add("swiglu fwd+bwd", lambda: torch.autograd.grad(F.gated_act(gu, "silu"), gu, go), (3 + 5) * T * Fm * 2)

    Tc = min(T, 8192)
    hid = torch.randn(Tc, D, device=dev).bfloat16().requires_grad_(True)
    w = (torch.randn(V, D, device=dev) * 0.02).bfloat16().requires_grad_(True)
    tgt = torch.randint(0, V, (Tc,), device=dev)
    flops = 3 * 2.0 * Tc * D * V

    def lce():
        loss, _ = F.linear_cross_entropy(hid, w, tgt, weight_is_vd=True, loss_scale=1.0 / Tc)
        return loss

    if not args.only or "cross" in args.only:
        ms = _time(lce, iters=5)
        rows.append({"kernel": f"linear_cross_entropy fwd+bwd ({Tc} rows x {V})", "ms": round(ms, 3),
                     "TFLOPs": round(flops / ms / 1e9, 1), "logit_bytes_never_in_HBM_GB": round(Tc * V * 4 / 1e9, 2)})

    C = 8192
    xc = torch.randn(B, S, C, device=dev).bfloat16().requires_grad_(True)
    wc = (torch.randn(C, 1, 4, device=dev) * 0.3).bfloat16().requires_grad_(True)
    with torch.no_grad():
        add("conv1d_silu_fwd (C=8192, K=4)", lambda: F.causal_conv1d_silu(xc, wc), 2 * xc.numel() * 2)
    gc = torch.randn_like(xc)
    add("conv1d_silu fwd+bwd", lambda: torch.autograd.grad(F.causal_conv1d_silu(xc, wc), (xc, wc), gc), 5 * xc.numel() * 2)

    check_status()
    for r in rows:
        print(json.dumps(r))
    if args.out:
        Path(args.out).write_text(json.dumps(rows, indent=1))


if __name__ == "__main__":
    main()
