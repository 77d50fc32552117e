#!/bin/bash
# Hardware calibration over several nodes (inter-node bandwidth rows of the g2g table).
#
#     HOSTS=host0,host1 bash mist_b200/tools/scripts/profile_interference_multinode.sh [gpus_per_node] [output_dir]
#
# The repository must sit at the same path on every host; host0 is the rendezvous address.  Each run writes
# one record file per layout on the first host; merge and fit as in the single-node script.
set -e
GPUS=${1:-8}
OUT=${2:-calibration}
: "${HOSTS:?set HOSTS=host0,host1,...}"
ROOT_PATH=$(pwd)
MASTER_ADDR=${HOSTS%%,*}
NUM_HOSTS=$(echo "${HOSTS}" | tr ',' '\n' | wc -l)
mkdir -p "${OUT}"

run_multinode_profiling() {
    GROUP=$1
    echo "--- ${NUM_HOSTS} hosts x ${GPUS} GPUs, group size ${GROUP} ---"
    pdsh -S -R ssh -w "${HOSTS}" \
        "cd ${ROOT_PATH} && python -m torch.distributed.run --nnodes ${NUM_HOSTS} --nproc-per-node ${GPUS} \
            --node-rank %n --master-addr ${MASTER_ADDR} --master-port 29612 \
            -m mist_b200.tools.profile_interference --group-sizes ${GROUP} \
            --out ${OUT}/bandwidth-n${NUM_HOSTS}-m${GPUS}-group${GROUP}.json >> ${OUT}/stdout.log 2>&1"
}

run_multinode_profiling $((NUM_HOSTS * GPUS))
run_multinode_profiling $((NUM_HOSTS * 2))
python -m mist_b200.tools.merge_json_results "${OUT}"/bandwidth-n*.json -o "${OUT}/bandwidth-merged.json"
python -m mist_b200.tools.comm_model "${OUT}/bandwidth-merged.json"
