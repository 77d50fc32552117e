#!/bin/bash
# Hardware calibration on one node: measures compute / collective / host-copy interference for groups of
# 8, 4 and 2 GPUs, merges the records and fits the parameter lists for the hardware template
# (g2g, c2g, g2c, interference).  Run from the repository root on the machine to calibrate:
#
#     bash mist_b200/tools/scripts/profile_interference_single_node.sh [gpus_per_node] [output_dir]
#
# Paste the four printed lists into the hardware block of the experiment template
# (mist_b200/configs/generate.py, then `python -m mist_b200.configs.generate`).
set -e
GPUS=${1:-8}
OUT=${2:-calibration}
mkdir -p "${OUT}"

run_profiling() {
    GROUP=$1
    python -m torch.distributed.run --nnodes=1 --nproc-per-node "${GPUS}" --master-addr 127.0.0.1 --master-port 29611 \
        -m mist_b200.tools.profile_interference --group-sizes "${GROUP}" \
        --out "${OUT}/bandwidth-n1-m${GPUS}-intra${GROUP}-inter1.json" >> "${OUT}/stdout.log" 2>&1
}

for g in 8 4 2; do
    if [ "${g}" -le "${GPUS}" ]; then run_profiling "${g}"; fi
done
python -m mist_b200.tools.merge_json_results "${OUT}"/bandwidth-n1-*.json -o "${OUT}/bandwidth-merged.json"
python -m mist_b200.tools.comm_model "${OUT}/bandwidth-merged.json"
