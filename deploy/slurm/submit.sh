#!/bin/bash
# A chain of dependent jobs for one run name; every link resumes where the previous one stopped.
#
#   bash deploy/slurm/submit.sh my-run                 # 1 node, 4 links of 24 h
#   NODES=8 LINKS=10 bash deploy/slurm/submit.sh my-run --override max_steps=200000
#   TIME=04:00:00 PARTITION=b200 ACCOUNT=proj bash deploy/slurm/submit.sh my-run
#   CONFIG=configs/finetune_768.yaml DATASETS="pdb:/data/pdb:0.5 distill:/data/distill:0.5::1" bash deploy/slurm/submit.sh ft
#
# Re-running with an existing run name appends links to that run (its frozen config is kept).
# (Reference: hangang/submit.sh.)
set -euo pipefail
HERE="$(cd "$(dirname "$0")" && pwd)"
RUN_NAME="${1:?usage: submit.sh RUN_NAME [train arguments...]}"
shift
export RUN_NAME EXTRA_ARGS="${*:-}"
args=(--parsable --nodes="${NODES:-1}" --time="${TIME:-24:00:00}" --job-name="df3-${RUN_NAME}" --export=ALL)
[[ -n "${PARTITION:-}" ]] && args+=(--partition="${PARTITION}")
[[ -n "${ACCOUNT:-}" ]] && args+=(--account="${ACCOUNT}")
prev="${AFTER:-}"
for link in $(seq "${LINKS:-4}"); do
  dep=()
  [[ -n "${prev}" ]] && dep=(--dependency="afterany:${prev}")
  prev="$(sbatch "${args[@]}" "${dep[@]}" "${HERE}/train.sbatch")"
  echo "link ${link}: job ${prev}"
done
echo "status: python -m deepfold3_dev_b200.cli run-status \${DF3_RUNS:-runs}/${RUN_NAME}"
