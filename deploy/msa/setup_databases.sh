#!/usr/bin/env bash
# Fetch and index the sequence databases of the local MSA pipeline (`msa --db-dir`, `msa-batch --db-dir`).
#
#   bash deploy/msa/setup_databases.sh /data/msa_dbs              # CPU search
#   GPU=1 bash deploy/msa/setup_databases.sh /data/msa_dbs        # also usable by the GPU prefilter / gpuserver
#   NO_INDEX=1 ...   skip the precomputed index (less disk, slower first search)
#   TEMPLATES=0 ...  skip the PDB sequence database used for template hits
#
# About 500 GB in all: uniref30_2302_db (UniRef30 clusters), colabfold_envdb_202108_db (environmental sequences),
# pdb100_230517 (PDB sequences). Every step leaves a `<name>.READY` stamp, so an interrupted run continues where it
# stopped. The databases and their names are those of ColabFold's public server; the reference prepares the same set
# (scripts/setup_databases.sh).
set -euo pipefail
DEST="${1:?usage: setup_databases.sh DIRECTORY}"
MMSEQS="${MMSEQS:-mmseqs}"
BASE="${BASE_URL:-https://wwwuser.gwdg.de/~compbiol/colabfold}"
THREADS="${THREADS:-$(nproc)}"
mkdir -p "${DEST}"; cd "${DEST}"
command -v "${MMSEQS}" >/dev/null || { echo "mmseqs not found (set MMSEQS=/path/to/mmseqs)" >&2; exit 1; }

fetch() {  # URL FILE
  [[ -f "$2" ]] && return 0
  if command -v aria2c >/dev/null; then aria2c --max-connection-per-server=8 --allow-overwrite=true -o "$2.part" "$1"
  else curl -L --fail --retry 5 -C - -o "$2.part" "$1"; fi
  mv "$2.part" "$2"
}

prepare() {  # NAME TARBALL
  local name="$1" tarball="$2"
  [[ -f "${name}.READY" ]] && { echo "${name}: ready"; return 0; }
  fetch "${BASE}/${tarball}" "${tarball}"
  tar xzf "${tarball}"
  "${MMSEQS}" tsv2exprofiledb "${name}" "${name}_db"
  if [[ "${GPU:-0}" == "1" ]]; then   # padded layout for the GPU prefilter; the CPU pipeline reads it too
    "${MMSEQS}" makepaddedseqdb "${name}_db" "${name}_db_pad"
    for f in "${name}_db_pad"*; do mv "$f" "${f/_db_pad/_db}"; done
  fi
  if [[ "${NO_INDEX:-0}" != "1" ]]; then
    "${MMSEQS}" createindex "${name}_db" tmp_index --remove-tmp-files 1 --threads "${THREADS}" ${GPU:+--index-subset 2}
  fi
  touch "${name}.READY"
}

prepare uniref30_2302 uniref30_2302.tar.gz
prepare colabfold_envdb_202108 colabfold_envdb_202108.tar.gz
if [[ "${TEMPLATES:-1}" == "1" && ! -f pdb100_230517.READY ]]; then
  fetch "${BASE}/pdb100_230517.fasta.gz" pdb100_230517.fasta.gz
  "${MMSEQS}" createdb pdb100_230517.fasta.gz pdb100_230517
  [[ "${NO_INDEX:-0}" == "1" ]] || "${MMSEQS}" createindex pdb100_230517 tmp_index --remove-tmp-files 1 --threads "${THREADS}"
  touch pdb100_230517.READY
fi
echo "databases under ${DEST}: $(ls *.READY | tr '\n' ' ')"
