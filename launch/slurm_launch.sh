#!/usr/bin/env bash
#SBATCH --job-name=mintext_b200
#SBATCH --nodes=2
#SBATCH --ntasks-per-node=1
#SBATCH --gpus-per-node=8
# Multi-node launch: one torchrun agent per node, one training process per GPU.
# The reference launcher's variables (JAX_COORDINATOR_IP/PORT, NNODES, NODE_RANK) are also exported because
# initialize_distributed() accepts them as aliases.
set -euo pipefail
export MASTER_ADDR="$(scontrol show hostnames "${SLURM_JOB_NODELIST}" | head -n 1)"
export MASTER_PORT="${MASTER_PORT:-29500}"
export JAX_COORDINATOR_IP="${MASTER_ADDR}" JAX_COORDINATOR_PORT="${MASTER_PORT}"
export NNODES="${SLURM_NNODES}"
srun bash -c 'export NODE_RANK=${SLURM_NODEID}; python -m torch.distributed.run \
  --nnodes ${NNODES} --node-rank ${NODE_RANK} --nproc-per-node ${GPUS_PER_NODE:-8} \
  --master-addr ${MASTER_ADDR} --master-port ${MASTER_PORT} -m mintext_b200.train '"$*"
