#!/bin/bash
# usage: submit.sh RUN_NAME [NODES] [LINKS]   -- a chain of LINKS dependent 24 h jobs for one run
set -euo pipefail
RUN_NAME="${1:?run name}"; NODES="${2:-1}"; LINKS="${3:-4}"
prev=""
for _ in $(seq "${LINKS}"); do
  dep=(); [[ -n "${prev}" ]] && dep=(--dependency="afterany:${prev}")
  prev=$(sbatch --parsable --nodes="${NODES}" --export=ALL,RUN_NAME="${RUN_NAME}" "${dep[@]}" "$(dirname "$0")/train.sbatch")
  echo "submitted ${prev}"
done
