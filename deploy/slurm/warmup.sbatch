#!/bin/bash
#SBATCH --job-name=df3-warmup
#SBATCH --nodes=1
#SBATCH --ntasks-per-node=1
#SBATCH --gres=gpu:1
#SBATCH --cpus-per-task=16
#SBATCH --time=00:30:00
#SBATCH --output=%x-%j.out
# Compile the sm_100a extension in-tree (once per checkout; the .so is then shared by every job through the file
# system) and run each kernel family once at the crop sizes of the run. The reference spends this job on filling its
# Triton autotune cache (hangang/warmup.sbatch); these kernels have nothing to tune, so this is a build + self-check.
set -euo pipefail
source "${SLURM_SUBMIT_DIR}/deploy/env.sh"
cd "${DF3_REPO}"
python -m deepfold3_dev_b200.ops.build
python -m deepfold3_dev_b200.cli warmup-kernels --tokens 384 --tokens 640 --tokens 768
python -c "import __graft_entry__ as e; e.smoke(); print('one training step: ok')"
