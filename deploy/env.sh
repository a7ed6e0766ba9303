# Shared environment for training on 8 x B200 nodes. Source it from a batch script or a container entry point:
#
#   source deploy/env.sh            # quiet defaults
#   DF3_COMM_LOG=1 source deploy/env.sh   # verbose collective logging for one diagnostic run
#
# The reference keeps the same knobs inside its site files (hangang/env.sh for Slurm + Slingshot,
# kakao/trainjob-multinode.yaml for Kubernetes + InfiniBand). They are gathered here once, site-neutral, so that the
# Slurm and Kubernetes recipes cannot drift apart. Everything can be overridden from the caller's environment.

# ---- paths -------------------------------------------------------------------------------------------------------
export DF3_REPO="${DF3_REPO:-$(cd "$(dirname "${BASH_SOURCE[0]}")/.." && pwd)}"
export DF3_DATA="${DF3_DATA:-/data}"                      # dataset root (packed or unpacked; loaders read both)
export DF3_RUNS="${DF3_RUNS:-${DF3_REPO}/runs}"           # run directories (checkpoints, logs, manifests)
export DF3_CACHE="${DF3_CACHE:-${HOME}/.cache/deepfold3-b200}"
mkdir -p "${DF3_CACHE}" 2>/dev/null || true

# ---- host side ---------------------------------------------------------------------------------------------------
# One process per GPU; the data threads and the featuriser share the remaining cores. Eight is enough to keep a B200
# fed at crop 384 (the input pipeline takes ~0.1 s of host time per example against a ~0.9 s step).
export OMP_NUM_THREADS="${OMP_NUM_THREADS:-8}"
export PYTHONUNBUFFERED=1
# Growable segments keep the caching allocator from fragmenting when crop sizes differ between steps.
export PYTORCH_CUDA_ALLOC_CONF="${PYTORCH_CUDA_ALLOC_CONF:-expandable_segments:True}"

# ---- inside a node: NVLink 5 / NVSwitch --------------------------------------------------------------------------
# The data-parallel optimizer step and the row-sharded trunk exchange over CUDA-IPC peer memory inside a node
# (DF3_COMM=peer, DF3_AXIAL_COMM=peer are the defaults on one node). With more than one node the gradient transport is
# NCCL (collective); say so explicitly so that a mis-detected topology fails loudly instead of silently degrading.
if [[ "${DF3_NODES:-1}" -gt 1 ]]; then
  export DF3_COMM="${DF3_COMM:-collective}"
fi
# NVLS (in-switch reduction) is left to NCCL's own detection. Turn it off only for elastic / rank-leave experiments:
# a rank that dies while its memory is bound to a multicast object takes its peers' GPUs with it.
# export NCCL_NVLS_ENABLE=0

# ---- between nodes: InfiniBand / RoCE ----------------------------------------------------------------------------
export NCCL_IB_DISABLE="${NCCL_IB_DISABLE:-0}"
# Pin the adapters that are cabled to the compute fabric. Auto-probing also finds storage / management adapters that
# cannot reach the peers, and NCCL then falls back to TCP without an error. The leading '=' asks for exact names.
# export NCCL_IB_HCA="=mlx5_0,mlx5_1,mlx5_2,mlx5_3,mlx5_4,mlx5_5,mlx5_6,mlx5_7"
# Interface for the bootstrap ring and the torch.distributed store (not the payload).
# export NCCL_SOCKET_IFNAME=eth0
# export GLOO_SOCKET_IFNAME=eth0

# ---- failure detection -------------------------------------------------------------------------------------------
# NCCL's RAS thread answers `ncclras` queries on a live job (which rank is behind, which communicator is stuck).
export NCCL_RAS_ENABLE="${NCCL_RAS_ENABLE:-1}"
# A collective that times out tears the process down instead of hanging the job; the flight recorder keeps the last
# collectives of every rank and dumps them on a timeout or on demand (write anything into the pipe file).
export TORCH_NCCL_ASYNC_ERROR_HANDLING="${TORCH_NCCL_ASYNC_ERROR_HANDLING:-1}"
export TORCH_FR_BUFFER_SIZE="${TORCH_FR_BUFFER_SIZE:-20000}"
export TORCH_NCCL_DUMP_ON_TIMEOUT="${TORCH_NCCL_DUMP_ON_TIMEOUT:-1}"
export TORCH_NCCL_DEBUG_INFO_PIPE_FILE="${TORCH_NCCL_DEBUG_INFO_PIPE_FILE:-/tmp/df3_fr_pipe}"
export TORCH_FR_DUMP_TEMP_FILE="${TORCH_FR_DUMP_TEMP_FILE:-/tmp/df3_fr_dump_}"
# The trainer's own guards (named collectives with a deadline, skip-together consensus, stop file) need no variable;
# the stop file is set per run by the launch recipe (DF3_STOP_FILE).

# ---- logging -----------------------------------------------------------------------------------------------------
if [[ "${DF3_COMM_LOG:-0}" == "1" ]]; then
  # Per-collective lines and transport timing, written to a node-local file so that the log itself does not load the
  # shared file system that is being diagnosed.
  export NCCL_DEBUG=INFO
  export NCCL_DEBUG_SUBSYS="${NCCL_DEBUG_SUBSYS:-INIT,NET,COLL}"
  export NCCL_DEBUG_FILE="${NCCL_DEBUG_FILE:-/tmp/nccl.%h.%p.log}"
  export TORCH_NCCL_ENABLE_TIMING=1
else
  export NCCL_DEBUG="${NCCL_DEBUG:-WARN}"
  export TORCH_NCCL_ENABLE_TIMING="${TORCH_NCCL_ENABLE_TIMING:-0}"
fi

df3_describe_env() {
  echo "repo=${DF3_REPO} data=${DF3_DATA} runs=${DF3_RUNS} nodes=${DF3_NODES:-1} comm=${DF3_COMM:-auto}"
  env | grep -E '^(NCCL_|TORCH_NCCL_|TORCH_FR_|DF3_)' | sort
}
