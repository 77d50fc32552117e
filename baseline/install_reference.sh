#!/bin/bash
# Installs the unmodified reference (Dazz993/Mist) under baseline/_ref for `bench.py --impl reference`.
#
#   bash baseline/install_reference.sh /path/to/reference [/path/to/wheelhouse]
#
# Step 1 is the plain offline pip install.  The reference's setup.py lists `packages=["mist"]` only, so
# pip copies the top-level modules and none of the sub-packages; step 2 completes the package by copying
# the remaining files of `mist/` byte for byte, together with the reference's exec driver and its YAML
# tree (they live outside the package, under benchmark/mist).  Step 3 writes a checksum listing and
# verifies that every file equals its source.  Nothing under baseline/_ref is edited.
set -euo pipefail
SRC=${1:?usage: install_reference.sh <reference checkout> [wheelhouse]}
WHEELS=${2:-/opt/wheelhouse}
HERE=$(cd "$(dirname "$0")" && pwd)
DST=$HERE/_ref
TMP=$(mktemp -d /tmp/mist_ref_src.XXXXXX)
cp -r "$SRC"/. "$TMP"/
rm -rf "$TMP/build" "$TMP/mist.egg-info"
rm -rf "$DST"
python -m pip install --no-index --no-build-isolation --no-deps --find-links "$WHEELS" \
    --target "$DST" "$TMP" 2>&1 | tail -2
# 2. the sub-packages setup.py leaves out, and the driver + configs
cp -r "$SRC/mist/." "$DST/mist/"
find "$DST" -name __pycache__ -type d -prune -exec rm -rf {} +
mkdir -p "$DST/benchmark/mist"
cp -r "$SRC/benchmark/mist/exec" "$DST/benchmark/mist/exec"
cp -r "$SRC/benchmark/mist/configs" "$DST/benchmark/mist/configs"
mkdir -p "$DST/csrc"
cp -r "$SRC/csrc/fused_dense_lib" "$DST/csrc/fused_dense_lib"
cp -r "$SRC/csrc/layer_norm" "$DST/csrc/layer_norm"
# 3. checksums: every copied file must equal its source
(cd "$DST" && find mist benchmark csrc -type f ! -name '*.pyc' -print0 | sort -z | xargs -0 sha256sum) > "$DST/SHA256SUMS"
(cd "$SRC" && find mist benchmark/mist/exec benchmark/mist/configs csrc/fused_dense_lib csrc/layer_norm -type f ! -name '*.pyc' ! -path '*/__pycache__/*' -print0 | sort -z | xargs -0 sha256sum) > "$TMP/SRC_SUMS"
if diff -q "$DST/SHA256SUMS" "$TMP/SRC_SUMS" > /dev/null; then
  echo "reference installed: $(wc -l < "$DST/SHA256SUMS") files, all identical to $SRC"
else
  echo "MISMATCH between $DST and $SRC"; diff "$DST/SHA256SUMS" "$TMP/SRC_SUMS" | head; exit 1
fi
rm -rf "$TMP"
