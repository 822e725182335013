"""Expert-parallel MoE expert stage (dispatch -> gate|up GEMM -> activation -> down GEMM -> combine), forward +
backward, on N GPUs of one node: the fused path (peer-store dispatch; expert GEMMs whose epilogues send the combine
and dispatch-gradient rows home over NVLink), the same exchange with separate pull kernels, and the NCCL baseline.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29700 \
        benchmarks/bench_ep.py [--experts 128 --hidden 2048 --inter 768 --topk 8 --tokens 16384] [--iters 5]

Times are CUDA events on every rank, maximum over ranks; FLOPs = 3 GEMM passes x 2 x tokens x topk x hidden x 3 x inter.
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


def main():
    ap = argparse.ArgumentParser()
    for k, v in (("experts", 128), ("hidden", 2048), ("inter", 768), ("topk", 8), ("tokens", 16384), ("iters", 5)):
        ap.add_argument(f"--{k}", type=int, default=v)
    a = ap.parse_args()
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from mintext_b200.ops._ext import check_status
    from mintext_b200.parallel import ep as ep_mod

    world, rank = dist.get_world_size(), dist.get_rank()
    El = a.experts // world
    g = torch.Generator(device="cpu").manual_seed(rank)
    x = torch.randn(a.tokens, a.hidden, generator=g).to(dev).bfloat16().requires_grad_(True)
    scores = torch.rand(a.tokens, a.experts, generator=g).to(dev)
    topk_w, topk_idx = torch.topk(scores, a.topk, dim=-1)
    topk_w = (topk_w / topk_w.sum(-1, keepdim=True)).bfloat16().requires_grad_(True)
    gw = torch.Generator(device="cpu").manual_seed(100 + rank)
    gate_up = (torch.randn(El, a.hidden, 2 * a.inter, generator=gw) * 0.02).to(dev).bfloat16().requires_grad_(True)
    down = (torch.randn(El, a.inter, a.hidden, generator=gw) * 0.02).to(dev).bfloat16().requires_grad_(True)
    dy = torch.randn(a.tokens, a.hidden, device=dev, dtype=torch.bfloat16)
    flops = 3 * 2.0 * a.tokens * a.topk * a.hidden * 3 * a.inter  # per rank (balanced routing)

    def run(kind):
        os.environ["MT_EP_FUSED_COMBINE"] = "0" if kind == "peer_unfused" else "1"
        ep = ep_mod.ExpertParallel(dist.group.WORLD, dev, 2.0, fused=kind != "collective")

        def step():
            if kind == "collective":
                y = ep_mod.experts_forward_collective(ep, x, topk_idx, topk_w, gate_up, down, "silu", a.experts, torch.bfloat16)
            else:
                y = ep_mod.experts_forward_peer(ep, x, topk_idx, topk_w, gate_up, down, "silu", a.experts)
            y.backward(dy)
            x.grad = topk_w.grad = gate_up.grad = down.grad = None

        for _ in range(3):
            step()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        dist.barrier()
        torch.cuda.synchronize()
        s.record()
        for _ in range(a.iters):
            step()
        e.record()
        torch.cuda.synchronize()
        t = torch.tensor([s.elapsed_time(e) / a.iters], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        check_status()
        if kind != "collective":
            ep.check_overflow()
        return float(t)

    out = {"world": world, "experts": a.experts, "hidden": a.hidden, "inter": a.inter, "topk": a.topk,
           "tokens_per_rank": a.tokens}
    for kind in ("peer_fused", "peer_unfused", "collective"):
        ms = run(kind)
        out[kind + "_ms"] = round(ms, 3)
        out[kind + "_tflops_per_gpu"] = round(flops / ms / 1e9, 1)
    if rank == 0:
        print(json.dumps(out), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
