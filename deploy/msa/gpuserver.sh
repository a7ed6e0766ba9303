#!/usr/bin/env bash
# Keep the MSA databases resident on GPUs: one `mmseqs gpuserver` per database, started once before a batch of
# searches. Searches run with `--gpu-server` (`msa --db-dir ... --gpu-server`) then skip the per-call load of the
# database onto the device.
#
#   bash deploy/msa/gpuserver.sh /data/msa_dbs start      # background processes, PIDs in /data/msa_dbs/gpuserver.pids
#   bash deploy/msa/gpuserver.sh /data/msa_dbs stop
#   UNIREF_GPUS=0,1 ENV_GPUS=2,3 PDB_GPUS=0 bash deploy/msa/gpuserver.sh /data/msa_dbs start
#
# On a B200 (180 GB) UniRef30 (about 60 GB padded) and the environmental database (about 110 GB) fit on one device each;
# give each its own device. (The reference starts the same servers in scripts/mmseqs_gpuserver.sh.)
set -euo pipefail
DB="${1:?usage: gpuserver.sh DB_DIR start|stop}"; CMD="${2:-start}"
MMSEQS="${MMSEQS:-mmseqs}"
PIDS="${DB}/gpuserver.pids"

serve() {  # DATABASE MAX_SEQS GPUS
  [[ -e "${DB}/$1.dbtype" || -e "${DB}/$1.idx.dbtype" ]] || { echo "skip $1: not in ${DB}"; return 0; }
  CUDA_VISIBLE_DEVICES="$3" nohup "${MMSEQS}" gpuserver "${DB}/$1" --max-seqs "$2" --db-load-mode 0 --prefilter-mode 1 \
      > "${DB}/gpuserver.$1.log" 2>&1 &
  echo "$!" >> "${PIDS}"
  echo "$1 on GPU(s) $3: pid $!"
}

case "${CMD}" in
start)
  : > "${PIDS}"
  serve uniref30_2302_db 10000 "${UNIREF_GPUS:-0}"
  serve colabfold_envdb_202108_db 10000 "${ENV_GPUS:-1}"
  serve pdb100_230517 300 "${PDB_GPUS:-0}"
  ;;
stop)
  [[ -f "${PIDS}" ]] || exit 0
  while read -r pid; do kill "${pid}" 2>/dev/null || true; done < "${PIDS}"
  rm -f "${PIDS}"
  ;;
*) echo "usage: gpuserver.sh DB_DIR start|stop" >&2; exit 2 ;;
esac
