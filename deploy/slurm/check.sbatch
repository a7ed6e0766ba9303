#!/bin/bash
#SBATCH --job-name=df3-check
#SBATCH --nodes=1
#SBATCH --ntasks-per-node=1
#SBATCH --gres=gpu:8
#SBATCH --cpus-per-task=96
#SBATCH --exclusive
#SBATCH --time=01:00:00
#SBATCH --output=%x-%j.out
# Pre-flight on one node before the first long job: GPUs, the sm_100a extension, collectives over NVLink (NCCL and the
# package's peer-memory kernels), dataset packs, and a timed pass through the real input pipeline.
#   sbatch deploy/slurm/check.sbatch                 # quick
#   CHECKSUMS=1 sbatch deploy/slurm/check.sbatch     # also compare every packed file with its source (reads all data)
# (Reference: hangang/check.sbatch + hangang/smoke_data.py.)
set -euo pipefail
source "${SLURM_SUBMIT_DIR}/deploy/env.sh"
cd "${DF3_REPO}"

echo "=== 1. GPUs"
nvidia-smi --query-gpu=index,name,memory.total,clocks.max.sm,power.limit --format=csv
python - <<'PY'
import torch
n = torch.cuda.device_count()
assert n == 8, f"expected 8 GPUs, found {n}"
cap = torch.cuda.get_device_capability(0)
assert cap == (10, 0), f"these kernels are built for sm_100a; device reports sm_{cap[0]}{cap[1]}"
print("cuda ok:", torch.cuda.get_device_name(0))
PY

echo "=== 2. extension and kernels"
python -m deepfold3_dev_b200.cli warmup-kernels --tokens 384
python -m deepfold3_dev_b200.cli bench-kernels --op gemm | tail -n 8

echo "=== 3. collectives inside the node"
python -m torch.distributed.run --standalone --local-addr 127.0.0.1 --nproc-per-node=8 \
    deploy/comm_check.py --peer --sizes-mib 1 64 1024 --min-busbw "${MIN_BUSBW:-400}"

echo "=== 4. dataset packs"
for pack in $(find "${DF3_DATA}" -maxdepth 4 -type d -name _pack 2>/dev/null); do
  shards=$(find "${pack}/shards" -name '*.tar' | wc -l)
  echo "${pack}: ${shards} shard(s)"
  if [[ "${CHECKSUMS:-0}" == "1" && -f "${pack}/SHA256SUMS" ]]; then (cd "${pack}" && sha256sum --quiet -c SHA256SUMS); fi
done
echo "files under ${DF3_DATA}: $(find "${DF3_DATA}" -type f | wc -l)"

echo "=== 5. input pipeline"
python deploy/slurm/smoke_data.py --config "${CONFIG:-configs/initial.yaml}" --examples "${EXAMPLES:-32}" \
    $(for spec in ${DATASETS:-pdb:${DF3_DATA}/pdb}; do echo --dataset "${spec}"; done)
echo "=== all checks passed"
