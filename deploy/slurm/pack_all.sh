#!/usr/bin/env bash
# Build a packed copy of the dataset tree for file systems with a file-count quota. For every dataset root the bulky
# subtrees (structures/, msa/, templates/, features/) go into `{root}/_pack/` (tar shards, sorted index and per-shard
# checksums, written by `python -m deepfold3_dev_b200.cli pack`); manifests, cluster tables and other small files are
# copied as they are. The datasets look for `{root}/_pack` by themselves, so configs only change their root path.
#
#   SRC=/store/df3/data DEST=/store/df3/packed bash deploy/slurm/pack_all.sh
#   ONLY="pdb distill/afdb" bash deploy/slurm/pack_all.sh          # some dataset roots only
#   VERIFY=0 bash deploy/slurm/pack_all.sh                          # skip the byte-for-byte check
#
# Resumable at two levels: a root whose pack carries a `.done` stamp is skipped, and an interrupted pack continues after
# its last finished shard. (Reference: hangang/pack_all.sh.)
set -euo pipefail
source "$(dirname "$0")/../env.sh"
SRC="${SRC:-${DF3_DATA}}"
DEST="${DEST:?set DEST to the packed staging directory}"
ROOTS="${ONLY:-pdb distill}"                                   # dataset roots, relative to SRC
BULKY="${BULKY:-structures/ msa/ templates/ features/}"        # subtrees of a root that go into its pack
mkdir -p "${DEST}"

for rel in ${ROOTS}; do
  src="${SRC}/${rel}"; out="${DEST}/${rel}/_pack"
  [[ -d "${src}" ]] || { echo "skip ${rel}: not in ${SRC}"; continue; }
  mkdir -p "${out}"
  if [[ -f "${out}/.done" ]]; then
    echo "done ${rel}"
  else
    echo "pack ${rel}"
    python -m deepfold3_dev_b200.cli pack --shard-size "${SHARD_BYTES:-8589934592}" \
        $(for p in ${BULKY}; do echo --include "${p}"; done) "${src}" "${out}"
    if [[ "${VERIFY:-1}" == "1" ]]; then
      python -m deepfold3_dev_b200.cli pack-verify --sample "${VERIFY_SAMPLE:-2000}" "${src}" "${out}"
    fi
    touch "${out}/.done"
  fi
  # everything of this root that is not in the pack
  (cd "${src}" && tar cf - $(for p in ${BULKY}; do echo --exclude="./${p%/}"; done) --exclude=_pack .) | (cd "${DEST}/${rel}" && tar xf -)
done
# files directly under SRC (component dictionary, caches)
find "${SRC}" -maxdepth 1 -type f -exec cp -p {} "${DEST}/" \;
echo "packed tree: $(find "${DEST}" -type f | wc -l) files, $(du -sh "${DEST}" | cut -f1)"
