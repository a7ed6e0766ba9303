#!/usr/bin/env bash
# End-to-end test of the walltime checkpoint with the real train.sbatch: two short linked jobs.
#
#   bash deploy/slurm/smoke_walltime.sh submit wt-test     # link 1: 30 min with USR1 15 min before the end; link 2: 15 min
#   bash deploy/slurm/smoke_walltime.sh check  wt-test     # after both have ended
#
# Link 1 must receive USR1, write a checkpoint at a step boundary and exit 0; link 2 must resume from that checkpoint
# and go on. The periodic checkpoint interval is pushed beyond the test, so a checkpoint on disk can only be the
# shutdown's. (Reference: hangang/smoke_walltime.sh.)
set -euo pipefail
HERE="$(cd "$(dirname "$0")" && pwd)"
source "${HERE}/../env.sh"
MODE="${1:?submit|check}"; RUN_NAME="${2:?run name}"
RUN_DIR="${DF3_RUNS}/${RUN_NAME}"; LOGS="${RUN_DIR}/slurm"

link() {  # TIME SIGNAL [sbatch arguments]
  local t="$1" sig="$2"; shift 2
  RUN_NAME="${RUN_NAME}" EXTRA_ARGS="--synthetic --override checkpoint_interval=1000000 --override eval_interval=1000000 ${EXTRA_ARGS:-}" \
    sbatch --parsable --nodes="${NODES:-2}" --time="${t}" --signal="${sig}" --job-name="df3-${RUN_NAME}" \
           --output="${LOGS}/%j.out" --export=ALL ${PARTITION:+--partition="${PARTITION}"} "$@" "${HERE}/train.sbatch"
}

case "${MODE}" in
submit)
  [[ ! -e "${RUN_DIR}" ]] || { echo "${RUN_DIR} exists; pick a new name" >&2; exit 1; }
  mkdir -p "${LOGS}"
  a="$(link 00:30:00 B:USR1@900)"
  b="$(link 00:15:00 B:USR1@300 --dependency="afterany:${a}")"
  echo "link 1: ${a}; link 2: ${b}; afterwards: smoke_walltime.sh check ${RUN_NAME}"
  ;;
check)
  mapfile -t logs < <(ls "${LOGS}"/*.out | sort -V)
  (( ${#logs[@]} == 2 )) || { echo "FAIL: expected 2 logs under ${LOGS}, found ${#logs[@]}" >&2; exit 1; }
  bad=0
  want()   { if grep -aqE "$3" "$2"; then echo "ok    $1"; else echo "FAIL  $1"; bad=1; fi; }
  unwant() { if grep -aqE "$3" "$2"; then echo "FAIL  $1"; bad=1; else echo "ok    $1"; fi; }
  want   "link 1 got USR1"                      "${logs[0]}" 'USR1: walltime near'
  want   "link 1 wrote the shutdown checkpoint" "${logs[0]}" 'stop requested: writing checkpoint at step [0-9]+'
  unwant "link 1 was not killed by Slurm"       "${logs[0]}" 'CANCELLED|DUE TO TIME LIMIT'
  want   "link 2 resumed"                       "${logs[1]}" 'resumed from .*checkpoint_[0-9]+\.pt at step [0-9]+'
  unwant "link 2 did not start from scratch"    "${logs[1]}" 'resumed from .* at step 0$'
  ls "${RUN_DIR}"/checkpoint_*.pt >/dev/null 2>&1 && echo "ok    checkpoint on disk" || { echo "FAIL  no checkpoint on disk"; bad=1; }
  exit "${bad}"
  ;;
*) echo "usage: smoke_walltime.sh submit|check RUN_NAME" >&2; exit 2 ;;
esac
