#!/bin/bash
# One node of 8 x B200 (180 GB): tune, analyze and execute each size.  Run from benchmark/mist_b200/experiment.
source ./scripts/base.sh

#   nnodes, nproc_per_node, model,  model_size, seq_len, global_batch_size, use_flash_attention, extra_args
run 1       2               "falcon"  "2.7b"      2048     16                 true
run 1       4               "falcon"  "7b"        2048     32                 true
run 1       8               "falcon"  "13b"       2048     128                true
run 1       8               "falcon"  "22b"       2048     64                 true
