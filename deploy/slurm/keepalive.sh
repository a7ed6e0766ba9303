#!/usr/bin/env bash
# Scratch file systems that purge by access time: report what is close to the limit under the data and run
# directories, and optionally refresh it.
#   bash deploy/slurm/keepalive.sh               # files not read for more than WARN_DAYS (default 10)
#   bash deploy/slurm/keepalive.sh --touch       # also refresh their access time
# Losing one tar shard of a pack makes every record inside unreadable, and training only touches the shards it samples
# from, so packs used for evaluation only (or a paused run) do age out. Check the site's policy before automating
# --touch; re-sending what was purged with transfer.sh is always allowed. (Reference: hangang/keepalive.sh.)
set -euo pipefail
source "$(dirname "$0")/../env.sh"
days="${WARN_DAYS:-10}"
for root in "${DF3_DATA}" "${DF3_RUNS}"; do
  [[ -d "${root}" ]] || continue
  stale=$(find "${root}" -type f -atime +"${days}" | wc -l)
  echo "${root}: ${stale} file(s) not read for more than ${days} days"
  if [[ "${1:-}" == "--touch" && "${stale}" -gt 0 ]]; then
    find "${root}" -type f -atime +"${days}" -exec touch -a -c {} +
    echo "${root}: access times refreshed"
  fi
done
