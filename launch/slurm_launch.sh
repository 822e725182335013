#!/usr/bin/env bash
#SBATCH --job-name=mintext_b200
#SBATCH --nodes=2
#SBATCH --ntasks-per-node=1
#SBATCH --gpus-per-node=8
# Multi-node launch: one torchrun agent per node, one training process per GPU.
# The reference launcher's variables (JAX_COORDINATOR_IP/PORT, NNODES, NODE_RANK) are also exported because
# initialize_distributed() accepts them as aliases.
# Lay the nodes out on the mesh with num_slices / dcn_*_parallelism, e.g. for 2 nodes of 8 GPUs:
#   sbatch launch/slurm_launch.sh --config configs/models/meta-llama-3-8b.yml num_slices=2 dcn_data_parallelism=2 \
#          ici_fsdp_parallelism=4 ici_tensor_parallelism=2
# (tensor- and expert-parallel groups that stay inside a node keep the peer-memory kernels; the optimizer step, which
# spans the nodes, composes NCCL collectives.)
set -euo pipefail
export MASTER_ADDR="$(scontrol show hostnames "${SLURM_JOB_NODELIST}" | head -n 1)"
export MASTER_PORT="${MASTER_PORT:-29500}"
export JAX_COORDINATOR_IP="${MASTER_ADDR}" JAX_COORDINATOR_PORT="${MASTER_PORT}"
export NNODES="${SLURM_NNODES}"
srun bash -c 'export NODE_RANK=${SLURM_NODEID}; python -m torch.distributed.run \
  --nnodes ${NNODES} --node-rank ${NODE_RANK} --nproc-per-node ${GPUS_PER_NODE:-8} \
  --master-addr ${MASTER_ADDR} --master-port ${MASTER_PORT} -m mintext_b200.train '"$*"
