"""Run a training config as a subprocess, parse the step log lines and write ``benchmark_results.json``
(reference: benchmarks/run_benchmark.py; this logger prints the ``MFU=`` token the parser keys on).

    python benchmarks/run_benchmark.py --config configs/benchmarks/llama-3.2-1b-b200.yml [--gpus 8] [--skip 2] [key=value ...]

``--warmup_steps`` and ``--extra_args k=v ...`` are the reference's spellings of ``--skip`` and the bare overrides.
"""

from __future__ import annotations

import argparse
import json
import re
import subprocess
import sys
from pathlib import Path

LINE = re.compile(r"step=(\d+) loss=([\d.eE+-]+) .*step_time=([\d.]+)s TFLOP/s/device=([\d.]+) tokens/s/device=([\d.]+) MFU=([\d.]+)%")


def parse(text: str, skip: int):
    rows = []
    for m in LINE.finditer(text):
        step = int(m.group(1))
        if step >= skip:
            rows.append({"step": step, "loss": float(m.group(2)), "step_time": float(m.group(3)),
                         "tflops_per_device": float(m.group(4)), "tokens_per_sec_per_device": float(m.group(5)),
                         "mfu_pct": float(m.group(6))})
    return rows


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", required=True)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--skip", "--warmup_steps", dest="skip", type=int, default=2,
                    help="leading steps excluded from the averages")
    ap.add_argument("--extra_args", nargs="*", default=[], help="further key=value overrides (also accepted bare)")
    ap.add_argument("--out", default="benchmark_results.json")
    args, rest = ap.parse_known_args()
    root = Path(__file__).resolve().parents[1]
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
           "--master-addr", "127.0.0.1", "--master-port", "29510", "-m", "mintext_b200.train", "--config", args.config, *args.extra_args, *rest]
    proc = subprocess.run(cmd, cwd=root, capture_output=True, text=True)
    rows = parse(proc.stdout + proc.stderr, args.skip)
    if not rows:
        print("No timed steps captured", file=sys.stderr)
        print((proc.stdout + proc.stderr)[-2000:], file=sys.stderr)
        sys.exit(1)
    mean = lambda k: sum(r[k] for r in rows) / len(rows)  # noqa: E731
    summary = {"config": args.config, "gpus": args.gpus, "timed_steps": len(rows), "step_time": mean("step_time"),
               "tflops_per_device": mean("tflops_per_device"), "tokens_per_sec_per_device": mean("tokens_per_sec_per_device"),
               "mfu_pct": mean("mfu_pct"), "steps": rows}
    Path(args.out).write_text(json.dumps(summary, indent=1))
    print(json.dumps({k: v for k, v in summary.items() if k != "steps"}))


if __name__ == "__main__":
    main()
