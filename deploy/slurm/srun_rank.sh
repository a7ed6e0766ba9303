#!/bin/bash
# Per-task wrapper under srun: translate Slurm's task variables into the ones torch.distributed reads, then exec the
# command. Every task sees all GPUs of its node and takes the one named by its local id (the package calls
# torch.cuda.set_device(LOCAL_RANK)); do not narrow CUDA_VISIBLE_DEVICES per task, or CUDA-IPC peer mappings between
# the tasks of a node stop working. (Reference: hangang/srun_rank.sh.)
export RANK="${SLURM_PROCID}" LOCAL_RANK="${SLURM_LOCALID}" WORLD_SIZE="${SLURM_NTASKS}"
export LOCAL_WORLD_SIZE="${SLURM_NTASKS_PER_NODE:-8}"
exec "$@"
