#!/bin/bash
# Executes every tuned configuration under a folder on the GPUs of this machine.
set -e
here="$(cd "$(dirname "$0")" && pwd)"
root="${1:-b200-180gb}"
gpus="${2:-8}"
for f in "$here/$root"/*/*.yaml; do
  name="$(basename "$f" .yaml)"
  echo "== $name"
  python -m torch.distributed.run --nnodes=1 --nproc-per-node "$gpus" --master-addr 127.0.0.1 \
    "$here/../exec/benchmark_one_case.py" -cd "$(dirname "$f")" --config-name "$name" output_dir="results/$root/$name"
done
