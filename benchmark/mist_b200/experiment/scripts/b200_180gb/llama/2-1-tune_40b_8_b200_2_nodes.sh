#!/bin/bash
# Two nodes: tuning and analysis only (CPU); the matching exec script runs the result.
source ./scripts/base.sh
run 2       8               "llama"  "40b"       2048     256                true                 "--skip-exec"
