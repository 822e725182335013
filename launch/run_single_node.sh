#!/usr/bin/env bash
# Train on the GPUs of one node, one process per GPU.
#   launch/run_single_node.sh <num_gpus> --config configs/models/meta-llama-3.2-1b.yml key=value ...
set -euo pipefail
NGPU="${1:?number of GPUs}"; shift
exec python -m torch.distributed.run --nnodes=1 --nproc-per-node "${NGPU}" \
  --master-addr 127.0.0.1 --master-port "${MASTER_PORT:-29500}" -m mintext_b200.train "$@"
