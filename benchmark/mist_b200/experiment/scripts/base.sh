#!/bin/bash
# Shared by the per-GPU experiment scripts: `run` tunes, analyzes and executes one case.
#
#   run <nnodes> <nproc_per_node> <model> <model_size> <seq_len> <global_batch_size> <use_flash_attention> [extra args]
#
# Run from benchmark/mist_b200/experiment.  Multi-node runs take the worker hosts from HOSTS
# (comma separated, first host = rendezvous address) and need the repository at the same path on every host.
ROOT_PATH=$(pwd)
LOG_DIR=${LOG_DIR:-logs}
case "${LOG_DIR}" in /*) LOG_ROOT="${LOG_DIR}" ;; *) LOG_ROOT="${ROOT_PATH}/${LOG_DIR}" ;; esac
EXPERIMENT=${EXPERIMENT:-template-b200}
SPACES=${SPACES:-mist}

run () {
  NUM_HOSTS=$1
  NUM_DEVICES_PER_HOST=$2
  MODEL_NAME=$3
  MODEL_SIZE=$4
  SEQ_LEN=$5
  GLOBAL_BATCH_SIZE=$6
  USE_FLASH_ATTENTION=$7
  EXTRA_ARGS=${8:-""}

  NUM_GPUS=$((NUM_HOSTS * NUM_DEVICES_PER_HOST))
  CASE_NAME=${MODEL_NAME}/${MODEL_SIZE}/N_${NUM_GPUS}-S_${SEQ_LEN}-B_${GLOBAL_BATCH_SIZE}-F_${USE_FLASH_ATTENTION}
  OUT_PATH=${LOG_ROOT}/${EXPERIMENT}/${CASE_NAME}
  mkdir -p "${OUT_PATH}"

  flash_attn=""
  if [ "${USE_FLASH_ATTENTION}" = false ]; then flash_attn="--disable-flash-attn"; fi
  hosts=""
  if [ "${NUM_HOSTS}" -gt 1 ] && [ -n "${HOSTS}" ]; then hosts="--hosts ${HOSTS}"; fi

  echo "--- ${CASE_NAME}: ${NUM_HOSTS} host(s) x ${NUM_DEVICES_PER_HOST} GPUs ---"
  echo "[TIME] before ${CASE_NAME}: $(date '+%Y-%m-%d-%H-%M-%S')" >> "${LOG_ROOT}/full_log.log"
  python run.py --model "${MODEL_NAME}/${MODEL_SIZE}" --experiment "${EXPERIMENT}" \
    --seq-len "${SEQ_LEN}" --global-batch-size "${GLOBAL_BATCH_SIZE}" \
    --nnodes "${NUM_HOSTS}" --nproc-per-node "${NUM_DEVICES_PER_HOST}" \
    --spaces ${SPACES} --out "${OUT_PATH}" ${flash_attn} ${hosts} ${EXTRA_ARGS} \
    2>&1 | tee -a "${OUT_PATH}/run.log"
  echo "[TIME] after  ${CASE_NAME}: $(date '+%Y-%m-%d-%H-%M-%S')" >> "${LOG_ROOT}/full_log.log"
}
