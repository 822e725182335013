"""Headline benchmark: training throughput of the Llama-3.2-1B-shaped model (bf16, global batch 64 x 4096,
AdamW, synthetic tokens, random init) on N GPUs of one node.  ``--model`` selects the other benchmark models
(`llama8b`: Llama-3-8B-shaped, FSDP 4 x TP 2, MXFP8 MLP GEMMs, 32 x 8192; `qwen3moe`: Qwen3-30B-A3B-shaped, EP 8,
32 x 4096; `dsv3`: DeepSeek-V3-shaped 4-layer MLA + MoE, EP 8, 16 x 4096), each read from
``configs/benchmarks/*.yml`` and set up exactly as ``python -m mintext_b200.train`` sets it up; ``--set key=value``
overrides config keys (e.g. a smaller expert count for a run on fewer GPUs).

    python bench.py --gpus 1 --steps K --warmup W
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W

Prints one JSON line (rank 0).  `value` is whole-job tokens/s, device-timed with CUDA events around exactly K
steps, max over ranks.  `e2e` repeats the measurement through the public engine API with the step's tokens
copied from pinned host memory and the loss read back to the host every step.
`--impl reference` reports whether the unmodified reference can run here.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

PUBLISHED_TOKENS_PER_SEC_PER_DEVICE = 22800.0  # reference's best published run (TPU v6e-8, Llama-3.2-1B)


def llama_1b_config(global_batch: int, seq_len: int, world: int, micro_batch: int, steps: int, fp8_mlp: bool = False,
                    fp8_recipe: str = "per_tensor"):
    from mintext_b200 import MinTextConfig

    per_rank = global_batch // world
    return MinTextConfig(
        model_name="llama-3.2-1b", model_type="llama3", num_hidden_layers=16, hidden_size=2048,
        num_attention_heads=32, num_key_value_heads=8, head_dim=64, intermediate_size=8192, vocab_size=128256,
        tie_word_embeddings=True, rope_theta=500000.0, rms_norm_eps=1e-5, seq_length=seq_len,
        per_device_batch_size=micro_batch, gradient_accumulation_steps=max(per_rank // micro_batch, 1),
        dtype="bfloat16", weight_dtype="float32", optimizer="adamw", learning_rate=3e-4, lr_schedule="cosine",
        steps=max(steps, 10), remat_policy="none", enable_tensorboard=False, enable_checkpointing=False,
        ici_fsdp_parallelism=world, use_fp8=fp8_mlp, fp8_recipe=fp8_recipe)


BENCH_MODELS = {
    # name: (config file, global batch in sequences, metric label, model description)
    "llama8b": ("llama-3-8b-b200.yml", 32, "train tokens/s (Llama-3-8B-shaped, FSDP x TP, AdamW)",
                "llama-3-8b-shaped (32L, d4096, 32/8 heads, ffn 14336, vocab 128256)"),
    "qwen3moe": ("qwen3-30b-a3b-b200.yml", 32, "train tokens/s (Qwen3-30B-A3B-shaped MoE, EP + FSDP, AdamW)",
                 "qwen3-30b-a3b-shaped (48L, d2048, 32/4 heads, 128 experts top-8, moe ffn 768, vocab 151936)"),
    "dsv3": ("deepseek-v3-4l-b200.yml", 16, "train tokens/s (DeepSeek-V3-shaped 4-layer MLA+MoE, EP + FSDP, AdamW)",
             "deepseek-v3-shaped 4 layers (d7168, MLA 128 heads, 256 experts top-8 + 1 shared, moe ffn 2048)"),
}


def yaml_config(name: str, world: int, global_batch: int | None, seq_len: int | None, micro_batch: int | None,
                steps: int, overrides: list[str]):
    """Config of one of the non-headline benchmark models with the batch split worked out for ``world`` ranks."""
    from mintext_b200.config import load_config, parse_cli_overrides

    yml, gb, _, _ = BENCH_MODELS[name]
    o = parse_cli_overrides(overrides) if overrides else {}
    if seq_len:
        o["seq_length"] = seq_len
    if micro_batch:
        o["per_device_batch_size"] = micro_batch
    o.update({"steps": max(steps, 10), "enable_tensorboard": False, "enable_checkpointing": False})
    cfg = load_config(ROOT / "configs" / "benchmarks" / yml, o)
    gb = global_batch or gb
    tp = max(int(cfg.ici_tensor_parallelism), 1)
    dp = world // tp
    if gb % dp != 0 or (gb // dp) % cfg.per_device_batch_size != 0:
        raise SystemExit(f"global batch {gb} does not split into {dp} data-parallel ranks x micro-batches of "
                         f"{cfg.per_device_batch_size}")
    return cfg.model_copy(update={"gradient_accumulation_steps": gb // dp // cfg.per_device_batch_size}), gb


class ClockSampler:
    """Samples SM clocks / throttle reasons with nvidia-smi while the timed region runs."""

    def __init__(self, index: int):
        self.index = index
        self.samples: list[tuple[float, float, str]] = []
        self._stop = threading.Event()
        self._t = threading.Thread(target=self._run, daemon=True)

    def _run(self):
        q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--query-gpu={q}", "--format=csv,noheader,nounits", "-i",
                                      str(self.index)], capture_output=True, text=True, timeout=5).stdout.strip()
                parts = [p.strip() for p in out.split(",")]
                reasons = [n for n, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown",
                                              "sw_power_cap"), parts[2:]) if v == "Active"]
                self.samples.append((float(parts[0]), float(parts[1]), ",".join(reasons)))
            except Exception:
                pass
            self._stop.wait(0.2)

    def __enter__(self):
        self._t.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        self._t.join(timeout=3)

    def summary(self) -> dict:
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        clocks = sorted(s[0] for s in self.samples)
        reasons = sorted({r for s in self.samples for r in s[2].split(",") if r})
        return {"sm_mhz": clocks[len(clocks) // 2], "sm_max_mhz": self.samples[0][1], "reasons": reasons,
                "samples": len(clocks)}


def run_reference(args) -> None:
    """The reference is a JAX program; report why it cannot run when its runtime is absent."""
    ref = ROOT / "baseline" / "_ref"
    why = None
    if not (ref / "mintext").exists():
        why = "reference package is not installed under baseline/_ref (offline pip install fails: dependency resolution needs the network)"
    else:
        sys.path.insert(0, str(ref))
        try:
            import mintext  # noqa: F401  (the unmodified reference)
            import mintext.train  # noqa: F401
        except Exception as e:
            why = ("reference installed with --no-deps but cannot be imported: its runtime (jax/flax/optax/orbax/grain/"
                   f"omegaconf) is not installed and not in the wheelhouse: {type(e).__name__}: {e}")
    if why is None:
        why = "reference imported, but no JAX CUDA backend is available to execute it on this image"
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": why.replace("\n", " ")[:400]}))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="own", choices=["own", "reference", "library"],
                    help="own: this framework; reference: the unmodified reference (reports why it cannot run here); "
                         "library: the same step composed from stock torch / cuBLAS / SDPA / NCCL pieces "
                         "(baseline/library_llama.py) - a same-box comparator, not the reference")
    ap.add_argument("--model", default="llama1b", choices=["llama1b"] + sorted(BENCH_MODELS))
    ap.add_argument("--global-batch", type=int, default=None)
    ap.add_argument("--seq-len", type=int, default=None)
    ap.add_argument("--micro-batch", type=int, default=None)
    ap.add_argument("--set", nargs="*", default=[], metavar="KEY=VALUE", help="config overrides (not for llama1b)")
    ap.add_argument("--skip-e2e", action="store_true")
    ap.add_argument("--profile-out", default=None, metavar="FILE",
                    help="after the measurement, run one more step under torch.profiler and write rank 0's "
                         "per-kernel time shares to FILE (outside every timed region)")
    ap.add_argument("--shard-params", action="store_true",
                    help="side measurement: layer weights and gradients sharded 1/N (fsdp_shard_params) instead of "
                         "resident on every rank; needs more than one GPU")
    ap.add_argument("--fp8-mlp", action="store_true",
                    help="side measurement, not the headline: MLP projections through the FP8 GEMM (per-tensor scales)")
    ap.add_argument("--fp8-recipe", choices=("per_tensor", "mx_block"), default="per_tensor",
                    help="with --fp8-mlp: per-tensor scales (e4m3 / e5m2) or MXFP8 block scales (e4m3, one scale per 32)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
        return

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
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}"

    from mintext_b200.models import Transformer
    from mintext_b200.parallel.engine import TrainEngine, local_batch_rows
    from mintext_b200.utils.pytree import model_flops_per_token_batch

    warmup = max(args.warmup, 3)
    if args.impl == "library":
        if args.model != "llama1b":
            raise SystemExit("--impl library covers the headline model only")
        sys.path.insert(0, str(ROOT / "baseline"))
        import library_llama

        args.global_batch = args.global_batch or 64
        args.seq_len = args.seq_len or 4096
        args.micro_batch = args.micro_batch or 8
        cfg = llama_1b_config(args.global_batch, args.seq_len, world, args.micro_batch, args.steps + warmup)
        eng = library_llama.LibraryTrainer(library_llama.LLAMA_1B, dev, world, args.micro_batch,
                                           total_steps=max(args.steps + warmup, 10))
        tp = 1
        metric = "train tokens/s (Llama-3.2-1B-shaped, bf16, AdamW)"
        model_desc = "llama-3.2-1b-shaped (16L, d2048, 32/8 heads, ffn 8192, vocab 128256, tied)"
        parallelism = eng.parallel
    elif args.model == "llama1b":
        args.global_batch = args.global_batch or 64
        args.seq_len = args.seq_len or 4096
        args.micro_batch = args.micro_batch or 8
        cfg = llama_1b_config(args.global_batch, args.seq_len, world, args.micro_batch, args.steps + warmup,
                              args.fp8_mlp, args.fp8_recipe)
        model = Transformer(cfg, rngs=0)
        if args.shard_params:
            from mintext_b200.parallel.fsdp import ParamShardedEngine

            eng = ParamShardedEngine(model, cfg.model_copy(update={"fsdp_shard_params": True}), device=dev)
        else:
            eng = TrainEngine(model, cfg, device=dev)
        tp = 1
        metric = "train tokens/s (Llama-3.2-1B-shaped, bf16, AdamW)"
        model_desc = "llama-3.2-1b-shaped (16L, d2048, 32/8 heads, ffn 8192, vocab 128256, tied)"
        parallelism = (f"fsdp{world}" if world > 1 else "single") + (" (parameters sharded)" if args.shard_params else "")
    else:
        from mintext_b200.train import setup_training

        cfg, args.global_batch = yaml_config(args.model, world, args.global_batch, args.seq_len, args.micro_batch,
                                             args.steps + warmup, args.set)
        args.seq_len, args.micro_batch = cfg.seq_length, cfg.per_device_batch_size
        mesh, model, eng, _, _ = setup_training(cfg)
        tp = mesh.shape["tensor"]
        _, _, metric, model_desc = BENCH_MODELS[args.model]
        parallelism = "x".join(f"{k}{v}" for k, v in (("fsdp", mesh.shape["data"] * mesh.shape["fsdp"]), ("tp", tp),
                                                       ("ep", mesh.shape["expert"])) if v > 1) or "single"
        if cfg.use_fp8:
            args.fp8_mlp, args.fp8_recipe = True, str(cfg.fp8_recipe)
    lo, hi = local_batch_rows(args.global_batch, world // tp, rank // tp)  # a tensor-parallel group shares its rows
    rows = hi - lo
    n_micro = max(rows // args.micro_batch, 1)
    gen = torch.Generator(device="cpu").manual_seed(1234 + rank // tp)

    def host_batch():
        t = torch.randint(0, cfg.vocab_size, (rows, args.seq_len), generator=gen, dtype=torch.int64)
        return t.pin_memory()

    # a pool of distinct batches, each far larger than nothing the L2 could keep between steps: one step streams
    # > 2.4 GB of weights and tens of GB of activations through a 126 MB L2, so no extra flush is needed
    dev_batches = [host_batch().to(dev, non_blocking=True) for _ in range(4)]

    def barrier_sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def step_device(i):
        tok = dev_batches[i % len(dev_batches)]
        return eng.train_step({"input_tokens": tok, "target_tokens": tok.roll(-1, dims=1)}, num_micro=n_micro)

    for i in range(warmup):
        out = step_device(i)
    barrier_sync()
    eng.check()
    launches_before = _count_launch_base(eng)
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as clocks:
        barrier_sync()
        start.record()
        for i in range(args.steps):
            out = step_device(i)
        end.record()
        barrier_sync()
    ms = start.elapsed_time(end)
    n_launches = _count_launches(eng, launches_before, args.steps)
    eng.check()
    t = torch.tensor([ms], device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    ms_per_step = ms / args.steps
    tokens_per_step = args.global_batch * args.seq_len
    value = tokens_per_step / (ms_per_step / 1e3)
    final_loss = float(out["loss"])

    # end-to-end: pinned host tokens -> device each step, loss read back each step
    e2e = None
    if not args.skip_e2e:
        hosts = [host_batch() for _ in range(4)]
        for i in range(2):
            tok = hosts[i % 4].to(dev, non_blocking=True)
            float(eng.train_step({"input_tokens": tok, "target_tokens": tok.roll(-1, dims=1)},
                                 num_micro=n_micro)["loss"])
        barrier_sync()
        s2, e2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s2.record()
        for i in range(args.steps):
            tok = hosts[i % 4].to(dev, non_blocking=True)
            o2 = eng.train_step({"input_tokens": tok, "target_tokens": tok.roll(-1, dims=1)}, num_micro=n_micro)
            final_loss = float(o2["loss"])  # device -> host read of the step's result
        e2.record()
        barrier_sync()
        t2 = torch.tensor([s2.elapsed_time(e2)], device=dev)
        if world > 1:
            dist.all_reduce(t2, op=dist.ReduceOp.MAX)
        ms2 = float(t2.item()) / args.steps
        e2e = {"value": tokens_per_step / (ms2 / 1e3), "unit": "tokens/s", "ms_per_step": ms2,
               "h2d_bytes_per_step": rows * args.seq_len * 8, "d2h_bytes_per_step": 4}

    from mintext_b200.parallel.ep import current_ep

    dropped = None  # routed rows that exceeded an expert rank's receive capacity (whole run, all ranks)
    if current_ep() is not None:
        d = torch.tensor([current_ep().dropped_rows()], device=dev, dtype=torch.int64)
        if world > 1:
            dist.all_reduce(d)
        dropped = int(d.item())
    free_b, total_b = torch.cuda.mem_get_info(dev)  # includes symmetric-memory and NCCL buffers
    peak = torch.tensor([max(torch.cuda.max_memory_reserved(dev), total_b - free_b) / 2 ** 30], device=dev)
    if world > 1:
        dist.all_reduce(peak, op=dist.ReduceOp.MAX)
    peak_gb = round(float(peak.item()), 2)
    flops_step = model_flops_per_token_batch(cfg, args.global_batch)
    tflops_per_gpu = flops_step / (ms_per_step / 1e3) / 1e12 / world
    if rank == 0:
        line = {
            "metric": metric, "value": value, "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": warmup, "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "strong",
            # the reference publishes a number for the Llama-3.2-1B run only
            "vs_baseline": value / (PUBLISHED_TOKENS_PER_SEC_PER_DEVICE * world) if args.model == "llama1b" else None,
            "dtype": ("bf16 (mxfp8 MLP projections)" if args.fp8_recipe == "mx_block" else "bf16 (fp8 e4m3/e5m2 MLP projections)") if args.fp8_mlp else ("bf16 (mxfp8 expert GEMMs)" if getattr(cfg, "moe_use_fp8", False) else "bf16"), "data": "synthetic uniform-random token ids, random-init weights", "impl": args.impl,
            "tokens_per_sec_per_gpu": value / world, "tflops_per_gpu": tflops_per_gpu,
            "mfu_vs_nominal_2250": tflops_per_gpu / 2250.0, "final_loss": final_loss,
            "peak_memory_gb": peak_gb, "moe_dropped_rows": dropped,
            "config": {"model": model_desc,
                       "global_batch": args.global_batch, "seq_len": args.seq_len,
                       "parallelism": parallelism, "remat_policy": str(cfg.remat_policy),
                       "micro_batch": args.micro_batch, "grad_accum_per_rank": n_micro,
                       "l2": "inputs and weights per step exceed L2 (126 MB) by >20x; no explicit flush"},
            "clocks": clocks.summary(), "e2e": e2e,
            # own arm: launches of this repository's kernels; library arm: none of them run, by construction
            "gpu_launches": int(n_launches) if args.impl == "own" else 0,
        }
        print(json.dumps(line))
    if args.profile_out:
        from mintext_b200.utils.profiling import kernel_share_table

        text = kernel_share_table(lambda: step_device(0), header=f"model={args.model} gpus={world} global_batch="
                                  f"{args.global_batch} micro_batch={args.micro_batch} n_micro={n_micro} "
                                  f"plain step {ms_per_step:.1f} ms")
        if rank == 0:
            Path(args.profile_out).parent.mkdir(parents=True, exist_ok=True)
            Path(args.profile_out).write_text(text + "\n")
    if world > 1:
        dist.destroy_process_group()


def _count_launch_base(eng):
    from mintext_b200.ops import launch_counter

    return launch_counter.count()


def _count_launches(eng, before, steps):
    from mintext_b200.ops import launch_counter

    return launch_counter.count() - before


if __name__ == "__main__":
    main()
