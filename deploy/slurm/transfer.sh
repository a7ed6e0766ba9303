#!/usr/bin/env bash
# Move the packed dataset to the cluster and results back, over one multiplexed SSH connection (sites with one-time
# passwords ask once).
#
#   REMOTE=user@datamover.cluster REMOTE_ROOT=/scratch/user/df3 bash deploy/slurm/transfer.sh connect
#   ... transfer.sh push       # parallel, resumable rsync of $DEST (from pack_all.sh) to $REMOTE_ROOT/data
#   ... transfer.sh verify     # sha256 of every pack on the remote side against SHA256SUMS
#   ... transfer.sh status     # what is missing remotely (dry run)
#   ... transfer.sh runs       # bring run directories (checkpoints, logs) back into ./runs
#   ... transfer.sh close
#
# (Reference: hangang/transfer.sh.)
set -euo pipefail
REMOTE="${REMOTE:?set REMOTE=user@host}"
REMOTE_ROOT="${REMOTE_ROOT:?set REMOTE_ROOT}"
DEST="${DEST:-./packed}"
SOCK="${HOME}/.ssh/df3-transfer-%r@%h"
SSH="ssh -o ControlPath=${SOCK} -o ControlMaster=auto -o ControlPersist=12h"
JOBS="${JOBS:-8}"

case "${1:?connect|push|verify|status|runs|close}" in
connect) ${SSH} -fN "${REMOTE}" && echo "connection up for 12 h" ;;
close)   ${SSH} -O exit "${REMOTE}" ;;
status)  rsync -a --dry-run --itemize-changes -e "${SSH}" "${DEST}/" "${REMOTE}:${REMOTE_ROOT}/data/" | grep -c '^<' || true ;;
push)
  ${SSH} "${REMOTE}" mkdir -p "${REMOTE_ROOT}/data"
  # directories and small files first, then the shards JOBS at a time; --partial lets a broken copy continue
  rsync -a --exclude='shards/' -e "${SSH}" "${DEST}/" "${REMOTE}:${REMOTE_ROOT}/data/"
  (cd "${DEST}" && find . -path '*/shards/*.tar' -print0) |
    xargs -0 -P "${JOBS}" -I{} rsync -a --partial --inplace --relative -e "${SSH}" "${DEST}/./{}" "${REMOTE}:${REMOTE_ROOT}/data/"
  echo "pushed; now: transfer.sh verify"
  ;;
verify)
  ${SSH} "${REMOTE}" "cd '${REMOTE_ROOT}/data' && find . -name SHA256SUMS -print0 | xargs -0 -n1 -P ${JOBS} sh -c 'cd \"\$(dirname \"\$0\")\" && sha256sum --quiet -c SHA256SUMS && echo ok \$(pwd)'"
  ;;
runs)
  mkdir -p runs
  rsync -a --partial -e "${SSH}" --include='*/' --include='checkpoint_*.pt' --include='*.yaml' --include='*.json*' \
        --include='*.log' --include='*.out' --exclude='*' "${REMOTE}:${REMOTE_ROOT}/runs/" runs/
  ;;
*) echo "unknown command $1" >&2; exit 2 ;;
esac
