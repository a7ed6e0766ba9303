#!/usr/bin/env bash
# Which pod and host owns which RDMA address.
#
#   bash deploy/k8s/rdma_ip_map.sh my-run > rdma_map.txt      # table for every pod of the job, while it is up
#   bash deploy/k8s/rdma_ip_map.sh my-run 10.1.64.7           # who owns this address?
#
# When NCCL cannot reach a peer at start-up it names the peer by the address of its secondary (Multus) interface. Those
# addresses are handed out per pod and are gone once the job is torn down, so take the table right after submitting and
# look the address up later. An address that maps to the same host over several submissions points at that host (add it
# to EXCLUDE_HOSTS); a different host every time points at a start-up race, and excluding hosts will not help.
# Same purpose as the reference's kakao/rdma_ip_map.sh; SUBNET is the prefix of the RDMA network (default 10.).
set -euo pipefail
JOB="${1:?usage: rdma_ip_map.sh JOB_NAME [ADDRESS]}"
WANTED="${2:-}"
NAMESPACE="${NAMESPACE:-default}"
KUBECTL="${KUBECTL:-kubectl -n ${NAMESPACE}}"
SUBNET="${SUBNET:-10.}"

${KUBECTL} get pods -o json | JOB="${JOB}" WANTED="${WANTED}" SUBNET="${SUBNET}" python3 -c "$(cat <<'PY'
import json, os, sys

job, wanted, subnet = os.environ["JOB"], os.environ["WANTED"], os.environ["SUBNET"]
table, owners = [], {}
for pod in json.load(sys.stdin)["items"]:
    meta, name = pod["metadata"], pod["metadata"]["name"]
    if not name.startswith(job):
        continue
    host = pod["spec"].get("nodeName", "-")
    state = pod.get("status", {}).get("phase", "-")
    try:
        nets = json.loads(meta.get("annotations", {}).get("k8s.v1.cni.cncf.io/network-status", "[]"))
    except ValueError:
        nets = []
    addrs = sorted({ip for net in nets for ip in net.get("ips", []) if ip.startswith(subnet) and not net.get("default")})
    for ip in addrs:
        owners[ip] = (host, name)
    table.append((name, host, state, addrs))
if not table:
    sys.exit(f"no pod of {job!r} found: the job is gone, and its addresses with it")
for name, host, state, addrs in sorted(table):
    print(f"{name:40s} {host:24s} {state:10s} {len(addrs):2d}  {' '.join(addrs) if addrs else '(none)'}")
if wanted:
    host, name = owners.get(wanted, (None, None))
    print()
    print(f"{wanted}: host {host}, pod {name}" if host else f"{wanted}: no pod of {job} owns it (old address, or an interface that never came up)")
PY
)"
