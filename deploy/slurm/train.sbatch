#!/bin/bash
#SBATCH --job-name=df3-b200
#SBATCH --ntasks-per-node=8
#SBATCH --gres=gpu:8
#SBATCH --cpus-per-task=12
#SBATCH --exclusive
#SBATCH --time=24:00:00
#SBATCH --signal=B:USR1@600
#SBATCH --output=%x-%j.out
# One srun task per GPU. RUN_NAME, CONFIG and DATA come from submit.sh.
set -euo pipefail
: "${RUN_NAME:?submit through deploy/slurm/submit.sh}"
REPO="${REPO:-$SLURM_SUBMIT_DIR}"
RUN_DIR="${RUNS:-$REPO/runs}/${RUN_NAME}"
mkdir -p "${RUN_DIR}"
# freeze the config on the first job of the chain so that a later edit cannot change a running experiment
[[ -f "${RUN_DIR}/config.yaml" ]] || cp "${CONFIG:-$REPO/configs/initial.yaml}" "${RUN_DIR}/config.yaml"

export MASTER_ADDR="$(scontrol show hostnames "${SLURM_JOB_NODELIST}" | head -n 1)"
export MASTER_PORT="${MASTER_PORT:-29500}"
export OMP_NUM_THREADS=8
export DF3_STOP_FILE="${RUN_DIR}/.stop-${SLURM_JOB_ID}"
# USR1 arrives 10 minutes before the walltime: ask the ranks to checkpoint and leave at a step boundary.
trap 'echo "walltime near: requesting checkpoint"; touch "${DF3_STOP_FILE}" || true' USR1

srun --kill-on-bad-exit=1 bash -c '
  export RANK=${SLURM_PROCID} LOCAL_RANK=${SLURM_LOCALID} WORLD_SIZE=${SLURM_NTASKS}
  exec python -m deepfold3_dev_b200.cli train --config "'"${RUN_DIR}"'/config.yaml" --output "'"${RUN_DIR}"'" \
       --dataset "pdb:'"${DATA:?set DATA}"'" --resume auto '"${EXTRA_ARGS:-}"'
' &
wait $!   # returns when the trap fires, too
wait
rm -f "${DF3_STOP_FILE}"
