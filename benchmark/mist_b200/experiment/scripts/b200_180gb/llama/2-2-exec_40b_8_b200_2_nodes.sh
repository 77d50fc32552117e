#!/bin/bash
# Two nodes: executes the strategy the tune script left behind.  HOSTS=host0,host1 must be set.
source ./scripts/base.sh
run 2       8               "llama"  "40b"       2048     256                true                 "--skip-tune"
