#!/usr/bin/env bash
# Batch-size sweep of the Llama-3.2-1B-shaped model (seq 4096, synthetic data), as the reference's
# scripts/benchmark_llama_1b.sh does on TPU.  Usage: launch/benchmark_llama_1b.sh [num_gpus]
set -euo pipefail
NGPU="${1:-1}"
for PDB in 1 4 8 16; do
  echo "=== per_device_batch_size=${PDB}"
  python -m torch.distributed.run --nnodes=1 --nproc-per-node "${NGPU}" --master-addr 127.0.0.1 \
    --master-port 29500 -m mintext_b200.train --config configs/benchmarks/llama-3.2-1b-b200.yml \
    per_device_batch_size="${PDB}" steps=20 run_name="bench_pdb${PDB}" 2>&1 | grep -E "step=(1[0-9])" || true
done
