#!/bin/bash
#SBATCH --job-name=df3-b200
#SBATCH --ntasks-per-node=8
#SBATCH --gres=gpu:8
#SBATCH --cpus-per-task=12
#SBATCH --exclusive
#SBATCH --time=24:00:00
#SBATCH --signal=B:USR1@600
#SBATCH --output=%x-%j.out
# One link of a training chain: one srun task per GPU. Submit through deploy/slurm/submit.sh, which sets RUN_NAME (and
# passes CONFIG, DATASETS, EXTRA_ARGS through). Ten minutes before the walltime Slurm sends USR1 to this script; the
# trap creates the stop file, every rank sees it at its next step boundary, the ranks agree to stop, rank 0 writes a
# checkpoint and the job exits 0. The next link resumes from that checkpoint (--resume auto).
# (Reference: hangang/train.sbatch does the same with its own trainer's signal handling.)
set -euo pipefail
: "${RUN_NAME:?submit through deploy/slurm/submit.sh}"
export DF3_NODES="${SLURM_JOB_NUM_NODES:-1}"
source "${SLURM_SUBMIT_DIR}/deploy/env.sh"
cd "${DF3_REPO}"
RUN_DIR="${DF3_RUNS}/${RUN_NAME}"
mkdir -p "${RUN_DIR}/slurm"
# freeze the config on the first link so that a later edit cannot change a running experiment
[[ -f "${RUN_DIR}/config.yaml" ]] || cp "${CONFIG:-${DF3_REPO}/configs/initial.yaml}" "${RUN_DIR}/config.yaml"

export MASTER_ADDR="$(scontrol show hostnames "${SLURM_JOB_NODELIST}" | head -n 1)"
export MASTER_PORT="${MASTER_PORT:-$((20000 + SLURM_JOB_ID % 20000))}"
export DF3_STOP_FILE="${RUN_DIR}/.stop-${SLURM_JOB_ID}"
DATASET_FLAGS=""
for spec in ${DATASETS:-pdb:${DF3_DATA}/pdb}; do DATASET_FLAGS+=" --dataset ${spec}"; done
df3_describe_env

trap 'echo "USR1: walltime near, asking the ranks to checkpoint and leave"; touch "${DF3_STOP_FILE}" || true' USR1
srun --kill-on-bad-exit=1 --cpu-bind=cores bash "${DF3_REPO}/deploy/slurm/srun_rank.sh" \
     python -m deepfold3_dev_b200.cli train --config "${RUN_DIR}/config.yaml" --output "${RUN_DIR}" \
     --resume auto ${DATASET_FLAGS} ${EXTRA_ARGS:-} &
step=$!
wait "${step}" || true      # returns early when the trap fires
wait "${step}"; rc=$?       # the real exit status of the step
rm -f "${DF3_STOP_FILE}"
exit "${rc}"
