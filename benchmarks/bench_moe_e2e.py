"""End-to-end MoE block benchmark, forward + backward (the reference's benchmarks/benchmark_moe_e2e.py shapes).

    python benchmarks/bench_moe_e2e.py [--shapes tiny,small,medium,dsv3_small]
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

SHAPES = {  # name: (experts, hidden, moe_intermediate, top_k, batch, seq)
    "tiny": (4, 128, 256, 2, 2, 128),
    "small": (8, 256, 512, 2, 4, 256),
    "medium": (16, 512, 1024, 4, 4, 512),
    "dsv3_small": (64, 512, 1024, 8, 4, 1024),
    "qwen3_30b_layer": (128, 2048, 768, 8, 4, 4096),
}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--shapes", default="small,medium,dsv3_small,qwen3_30b_layer")
    args = ap.parse_args()
    from mintext_b200 import MinTextConfig
    from mintext_b200.modules import MoEBlock

    for name in args.shapes.split(","):
        E, D, I, K, B, S = SHAPES[name]
        groups = 8 if E % 8 == 0 and E >= 64 else 1
        cfg = MinTextConfig(hidden_size=D, num_experts=E, num_experts_per_tok=K, moe_intermediate_size=I, n_group=groups,
                            topk_group=max(groups // 2, 1), n_shared_experts=1)
        blk = MoEBlock(cfg, rngs=torch.Generator().manual_seed(0)).cuda()
        for p in blk.parameters():
            if p.dim() >= 2:
                p.data = p.data.bfloat16()
        x = torch.randn(B, S, D, device="cuda", dtype=torch.bfloat16, requires_grad=True)

        def step():
            out, _ = blk(x)
            out.float().mean().backward()
            for p in blk.parameters():
                p.grad = None
            x.grad = None

        for _ in range(3):
            step()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        s.record()
        for _ in range(5):
            step()
        e.record()
        torch.cuda.synchronize()
        ms = s.elapsed_time(e) / 5
        flops = 3 * (2.0 * B * S * D * E + K * 2.0 * B * S * D * I * 3 + 2.0 * B * S * D * I * 3)
        print(json.dumps({"shape": name, "tokens": B * S, "fwd_bwd_ms": round(ms, 3), "tflops": round(flops / ms / 1e9, 1)}))


if __name__ == "__main__":
    main()
