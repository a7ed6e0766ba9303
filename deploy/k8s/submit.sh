#!/usr/bin/env bash
# Render deploy/k8s/trainjob-multinode.yaml and submit it.
#
#   bash deploy/k8s/submit.sh                                  # run name df3-YYYYMMDD-HHMMSS, 8 nodes
#   NODES=2 bash deploy/k8s/submit.sh my-run
#   bash deploy/k8s/submit.sh my-run --override max_steps=50000 --override alpha_pae=1.0
#   DATASETS="pdb:/data/pdb:0.5 distill:/data/distill:0.5::1" bash deploy/k8s/submit.sh my-run
#   DF3_COMM_LOG=1 bash deploy/k8s/submit.sh my-run            # verbose collective logs in /tmp of every pod
#   EXCLUDE_HOSTS=host-a,host-b bash deploy/k8s/submit.sh my-run
#   DRY_RUN=1 bash deploy/k8s/submit.sh my-run                 # print the rendered manifest, submit nothing
#
# Re-submitting an existing run name resumes it: the frozen config and the newest checkpoint in /runs/<name> are used.
# The reference's submitter (kakao/submit.sh) fills its template the same way; the knobs here are the ones a B200 /
# InfiniBand cluster needs, with no site names baked in.
set -euo pipefail
HERE="$(cd "$(dirname "$0")" && pwd)"
TEMPLATE="${TEMPLATE:-${HERE}/trainjob-multinode.yaml}"
NAMESPACE="${NAMESPACE:-default}"
KUBECTL="${KUBECTL:-kubectl -n ${NAMESPACE}}"

RUN_NAME="${1:-df3-$(date +%Y%m%d-%H%M%S)}"
shift || true
EXTRA_ARGS="${*:-}"
NODES="${NODES:-8}"
(( NODES >= 1 )) || { echo "NODES must be >= 1" >&2; exit 2; }
JOB_NAME="$(echo "${RUN_NAME}" | tr '[:upper:]_.' '[:lower:]--' | cut -c1-50)"   # DNS label
DATASET_FLAGS=""
for spec in ${DATASETS:-pdb:/data/pdb}; do DATASET_FLAGS+=" --dataset ${spec}"; done
ADAPTERS="${ADAPTERS:-8}"
RDMA_NETWORK="${RDMA_NETWORK:-rdma-net}"
NETWORKS="${RDMA_NETWORK}"
for _ in $(seq 2 "${ADAPTERS}"); do NETWORKS+=",${RDMA_NETWORK}"; done
EXCLUDE="$(echo "${EXCLUDE_HOSTS:-none}" | sed 's/[^,][^,]*/"&"/g')"

render() {
  sed -e "s|__JOB_NAME__|${JOB_NAME}|g" -e "s|__RUN_NAME__|${RUN_NAME}|g" \
      -e "s|__NODES__|${NODES}|g" -e "s|__WORKERS__|$((NODES - 1))|g" \
      -e "s|__RESTARTS__|${RESTARTS:-3}|g" -e "s|__IMAGE__|${IMAGE:-registry.local/deepfold3-b200:latest}|g" \
      -e "s|__CONFIG__|${CONFIG:-configs/initial.yaml}|g" -e "s|__DATASETS__|${DATASET_FLAGS}|g" \
      -e "s|__EXTRA_ARGS__|${EXTRA_ARGS}|g" -e "s|__COMM_LOG__|${DF3_COMM_LOG:-0}|g" \
      -e "s|__IB_HCA__|${IB_HCA:-}|g" -e "s|__SOCKET_IFNAME__|${SOCKET_IFNAME:-eth0}|g" \
      -e "s|__RDMA_NETWORKS__|${NETWORKS}|g" -e "s|__RDMA_RESOURCE__|${RDMA_RESOURCE:-rdma/hca}|g" \
      -e "s|__EXCLUDE_HOSTS__|${EXCLUDE}|g" -e "s|__DATA_PVC__|${DATA_PVC:-df3-data}|g" \
      -e "s|__RUNS_PVC__|${RUNS_PVC:-df3-runs}|g" -e "s|__WANDB_PROJECT__|${WANDB_PROJECT:-deepfold3-b200}|g" \
      -e "s|__WANDB_ENTITY__|${WANDB_ENTITY:-}|g" "${TEMPLATE}"
}

if [[ "${DRY_RUN:-0}" == "1" ]]; then render; exit 0; fi
left="$(render | grep -o '__[A-Z_]*__' | sort -u || true)"
[[ -z "${left}" ]] || { echo "unfilled template tokens: ${left}" >&2; exit 2; }
# a finished or failed job of the same name has to go before the name can be reused
${KUBECTL} delete pytorchjob "${JOB_NAME}" --ignore-not-found --wait=true
render | ${KUBECTL} apply -f -
cat <<MSG
submitted ${JOB_NAME} (${NODES} x 8 GPUs), run directory /runs/${RUN_NAME}
  logs     ${KUBECTL} logs -f ${JOB_NAME}-master-0
  stop     ${KUBECTL} exec ${JOB_NAME}-master-0 -- touch /runs/${RUN_NAME}/.stop     # checkpoint, then exit
  status   ${KUBECTL} exec ${JOB_NAME}-master-0 -- python -m deepfold3_dev_b200.cli run-status /runs/${RUN_NAME}
  stragglers  ${KUBECTL} exec ${JOB_NAME}-master-0 -- ncclras
  collective dump  ${KUBECTL} exec POD -- bash -c 'echo 1 > /tmp/df3_fr_pipe'   # flight recorder -> /tmp/df3_fr_dump_<rank>
  rdma map  bash deploy/k8s/rdma_ip_map.sh ${JOB_NAME}
MSG
