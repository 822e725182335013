"""Tensor-parallel projection benchmark: all-gather -> GEMM and GEMM -> reduce-scatter as one kernel each over NVLink
peer memory, against the NCCL collective + GEMM composition, for one transformer layer's shapes.

Launch one process per GPU:
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29700 \
        benchmarks/bench_tp_gemm.py [--tokens 32768 --hidden 2048 --ffn 8192] [--out file.json]
Times are CUDA-event times, maximum over ranks.  Roofline per op: the slower of FLOPs / measured GEMM peak and
bytes that must cross NVLink / 770 GB/s.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))


def _time(fn, dev, iters=10, warmup=3):
    for _ in range(warmup):
        fn()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize(dev)
    dist.barrier()
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    torch.cuda.synchronize(dev)
    t = torch.tensor([s.elapsed_time(e) / iters], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=32768)
    ap.add_argument("--hidden", type=int, default=2048)
    ap.add_argument("--ffn", type=int, default=8192)
    ap.add_argument("--gemm-tflops", type=float, default=1400.0, help="measured bf16 GEMM peak for the roofline")
    ap.add_argument("--link-gbs", type=float, default=770.0)
    ap.add_argument("--out", default="")
    args = ap.parse_args()
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from mintext_b200.ops._ext import check_status
    from mintext_b200.parallel import tp as tpm

    t = dist.get_world_size()
    rank = dist.get_rank()
    fused = tpm.TensorParallel(dist.group.WORLD, dev, fused=True)
    plain = tpm.TensorParallel(dist.group.WORLD, dev, fused=False)
    T, D, Fl = args.tokens, args.hidden, args.ffn // t
    Tl = T // t
    x_local = torch.randn(Tl, D, device=dev).bfloat16()
    w_up = (torch.randn(D, Fl, device=dev) * 0.02).bfloat16()
    h = torch.randn(T, Fl, device=dev).bfloat16()
    w_down = (torch.randn(Fl, D, device=dev) * 0.02).bfloat16()
    rows = []
    with torch.no_grad():
        for name, fn_f, fn_p, flops, link_bytes in (
            ("all-gather -> GEMM (MLP up)", lambda: tpm.column_linear(x_local, [w_up], fused, torch.bfloat16),
             lambda: tpm.column_linear(x_local, [w_up], plain, torch.bfloat16), 2.0 * T * D * Fl,
             (t - 1) * Tl * D * 2),
            ("GEMM -> reduce-scatter (MLP down)", lambda: tpm.row_linear(h, w_down, fused, torch.bfloat16),
             lambda: tpm.row_linear(h, w_down, plain, torch.bfloat16), 2.0 * T * Fl * D, (t - 1) * Tl * D * 2),
        ):
            ms_f = _time(fn_f, dev)
            ms_p = _time(fn_p, dev)
            floor_ms = max(flops / (args.gemm_tflops * 1e12), link_bytes / (args.link_gbs * 1e9)) * 1e3
            rows.append({"op": name, "tp": t, "tokens": T, "hidden": D, "ffn_local": Fl, "fused_ms": round(ms_f, 4),
                         "nccl_ms": round(ms_p, 4), "speedup": round(ms_p / ms_f, 3), "roofline_ms": round(floor_ms, 4),
                         "fused_frac_of_roofline": round(floor_ms / ms_f, 3)})
    # fully sharded weight (FSDP): gather of W [D, F] folded into x @ W, vs all_gather_into_tensor + GEMM
    from mintext_b200.ops import tp_gemm
    from mintext_b200.ops._ext import ext, status_word

    Ff = args.ffn
    w_full = (torch.randn(D, Ff, device=dev) * 0.02).bfloat16()
    sw = tp_gemm.ShardedWeight(w_full, dist.group.WORLD, dev)
    xs = torch.randn(Tl, D, device=dev).bfloat16()
    wbuf = torch.empty(D, Ff, device=dev, dtype=torch.bfloat16)
    ybuf = torch.empty(Tl, Ff, device=dev, dtype=torch.bfloat16)

    def nccl_path():
        dist.all_gather_into_tensor(wbuf, sw.shard.detach())
        ext().gemm(xs, wbuf, ybuf, False, True, False, status_word(dev))

    with torch.no_grad():
        ms_f = _time(lambda: tp_gemm.fsdp_linear(xs, sw), dev)
        ms_p = _time(nccl_path, dev)
    flops, link_bytes = 2.0 * Tl * D * Ff, (t - 1) * (D // t) * Ff * 2
    floor_ms = max(flops / (args.gemm_tflops * 1e12), link_bytes / (args.link_gbs * 1e9)) * 1e3
    rows.append({"op": "FSDP weight all-gather -> GEMM (MLP up, full width)", "tp": t, "tokens": Tl, "hidden": D,
                 "ffn_local": Ff, "fused_ms": round(ms_f, 4), "nccl_ms": round(ms_p, 4), "speedup": round(ms_p / ms_f, 3),
                 "roofline_ms": round(floor_ms, 4), "fused_frac_of_roofline": round(floor_ms / ms_f, 3)})
    check_status(dev)
    if rank == 0:
        for r in rows:
            print(json.dumps(r))
        if args.out:
            Path(args.out).write_text(json.dumps(rows, indent=1))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
