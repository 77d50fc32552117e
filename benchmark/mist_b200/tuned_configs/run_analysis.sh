#!/bin/bash
# Predicted iteration time and peak memory of every tuned configuration under a folder (CPU only).
set -e
here="$(cd "$(dirname "$0")" && pwd)"
root="${1:-b200-180gb}"
for f in "$here/$root"/*/*.yaml; do
  name="$(basename "$f" .yaml)"
  echo "== $name"
  python "$here/../analysis/run.py" -cd "$(dirname "$f")" --config-name "$name" output_dir="results/$root/$name" | grep -E "Total latency|peak"
done
