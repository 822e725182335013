"""Per-kernel time shares of one training step of a benchmark model (torch.profiler, CUDA activities).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        benchmarks/profile_step.py --model qwen3moe --gpus N [--global-batch B] [--set key=value ...] [--out FILE]

Sets the model up as ``bench.py --model`` does, runs two warm-up steps and profiles one.  Rank 0 prints (and
optionally writes) a table of the kernels by total device time, the step's wall time, the sum of kernel time (how
busy the GPU was) and the number of launches.  Times under the profiler are for shares, not for reporting.
"""

from __future__ import annotations

import argparse
import os
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))


def main() -> None:
    import bench

    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="qwen3moe", choices=["llama1b"] + sorted(bench.BENCH_MODELS))
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--global-batch", type=int, default=None)
    ap.add_argument("--seq-len", type=int, default=None)
    ap.add_argument("--micro-batch", type=int, default=None)
    ap.add_argument("--set", nargs="*", default=[])
    ap.add_argument("--top", type=int, default=40)
    ap.add_argument("--out", default=None)
    args = ap.parse_args()

    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    from mintext_b200.parallel.engine import local_batch_rows

    if args.model == "llama1b":
        from mintext_b200.models import Transformer
        from mintext_b200.parallel.engine import TrainEngine

        gb, seq, mb = args.global_batch or 64, args.seq_len or 4096, args.micro_batch or 8
        cfg = bench.llama_1b_config(gb, seq, world, mb, 10)
        eng = TrainEngine(Transformer(cfg, rngs=0), cfg, device=dev)
        tp = 1
    else:
        from mintext_b200.train import setup_training

        cfg, gb = bench.yaml_config(args.model, world, args.global_batch, args.seq_len, args.micro_batch, 10, args.set)
        mesh, _, eng, _, _ = setup_training(cfg)
        tp = mesh.shape["tensor"]
    lo, hi = local_batch_rows(gb, world // tp, rank // tp)
    n_micro = max((hi - lo) // cfg.per_device_batch_size, 1)
    tok = torch.randint(0, cfg.vocab_size, (hi - lo, cfg.seq_length), device=dev)
    batch = {"input_tokens": tok, "target_tokens": tok.roll(-1, dims=1)}
    for _ in range(2):
        eng.train_step(batch, num_micro=n_micro)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    t0 = time.time()
    eng.train_step(batch, num_micro=n_micro)
    torch.cuda.synchronize()
    plain_ms = (time.time() - t0) * 1e3
    from mintext_b200.utils.profiling import kernel_share_table

    text = kernel_share_table(lambda: eng.train_step(batch, num_micro=n_micro), top=args.top,
                              header=f"model={args.model} gpus={world} global_batch={gb} micro_batch="
                                     f"{cfg.per_device_batch_size} n_micro={n_micro} overrides={args.set}\n"
                                     f"step without profiler: {plain_ms:.1f} ms")
    eng.check()
    if rank == 0:
        print(text)
        if args.out:
            Path(args.out).parent.mkdir(parents=True, exist_ok=True)
            Path(args.out).write_text(text + "\n")
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
