#!/usr/bin/env bash
# Llama training with parallelism hot switching on one node.
#
#   bash llama_hot_switch.sh [MODEL_SIZE=7b] [SEQ_LEN=32768] [NUM_GPUS=8] [STEPS=50] [DATASET=synthetic|commoncrawl|github]
#
# The strategy sets per (model, GPUs, context length, dataset) are the ones the reference's scripts use
# (hotspa/scripts/llama_hot_switch.sh:42-82, hotspa/scripts/exprs_for_paper/llama_hot_switch.sh); they are written
# in the reference's order: the strategy of the longest bucket first, then from the shortest bucket up.  A json
# dataset is read when DATA_ROOT holds web/refinedweb0.json (or github/...), vocab.json and merges.txt; otherwise the
# batches are synthetic (lognormal lengths, 32K tokens per GPU and step).
set -euo pipefail

MODEL_SIZE=${1:-7b}
SEQ_LEN=${2:-32768}
NUM_GPUS=${3:-8}
STEPS=${4:-50}
DATASET=${5:-synthetic}
GLOBAL_BATCH_SIZE=${GLOBAL_BATCH_SIZE:-512}
DATA_ROOT=${DATA_ROOT:-data}
MASTER_PORT=${MASTER_PORT:-29500}

case "${SEQ_LEN}" in
  32768) BUCKET_SIZES="32768 16384 4096 0" ;;
  16384) BUCKET_SIZES="16384 4096 0" ;;
  8192)  BUCKET_SIZES="8192 4096 0" ;;
  4096)  BUCKET_SIZES="4096 0" ;;
  *) echo "unsupported context length ${SEQ_LEN}"; exit 1 ;;
esac
N_BUCKETS=$(( $(echo ${BUCKET_SIZES} | wc -w) - 1 ))

# strategies for the 32K bucket set (three buckets); shorter contexts take a suffix of the list
KEY="${MODEL_SIZE}-${NUM_GPUS}-${DATASET}"
if [ "${SEQ_LEN}" != "32768" ] && [ "${DATASET}" = "github" ]; then KEY="${MODEL_SIZE}-${NUM_GPUS}-commoncrawl"; fi   # the 4-strategy sets are 32K ones
case "${KEY}" in
  7b-8-github)        STRATEGIES="1,4,2 8,1,1 4,2,1 2,2,2"; BUCKET_SIZES="32768 16384 8192 4096 0"; N_BUCKETS=4 ;;
  3b-8-*|7b-8-*)      STRATEGIES="1,4,2 8,1,1 2,2,2" ;;
  13b-8-github)       STRATEGIES="1,8,1 4,2,1 2,2,2 1,4,2"; BUCKET_SIZES="32768 16384 8192 4096 0"; N_BUCKETS=4 ;;
  13b-8-*)            STRATEGIES="1,8,1 4,2,1 1,4,2" ;;
  *-4-*)              STRATEGIES="1,4,1 4,1,1 2,2,1" ;;
  *-2-*)              STRATEGIES="1,2,1 2,1,1"; if [ "${N_BUCKETS}" -gt 2 ]; then BUCKET_SIZES="${SEQ_LEN} 4096 0"; N_BUCKETS=2; fi ;;
  *-1-*)              STRATEGIES="1,1,1"; BUCKET_SIZES="${SEQ_LEN} 0"; N_BUCKETS=1 ;;
  *) echo "no strategy table entry for ${KEY}"; exit 1 ;;
esac
if [ "${N_BUCKETS}" -lt "$(echo ${STRATEGIES} | wc -w)" ]; then
  # fewer buckets than strategies: keep the home strategy of the reference's shorter-context rows
  case "${N_BUCKETS}" in
    2) STRATEGIES="$(echo ${STRATEGIES} | awk '{print $NF, $2}')" ;;
    1) STRATEGIES="$(echo ${STRATEGIES} | awk '{print $2}')" ;;
  esac
fi

DATA_ARGS=""
case "${DATASET}" in
  commoncrawl) JSON=${DATA_ROOT}/web/refinedweb0.json ;;
  github)      JSON=${DATA_ROOT}/github/github0.json ;;
  *)           JSON="" ;;
esac
if [ -n "${JSON}" ] && [ -f "${JSON}" ]; then
  DATA_ARGS="--json_file ${JSON} --json_key content --vocab_file ${DATA_ROOT}/vocab.json --merge_file ${DATA_ROOT}/merges.txt --global_batch_size ${GLOBAL_BATCH_SIZE} --dataset ${DATASET}"
fi

export HETU_SWITCH_ALGORITHM=${HETU_SWITCH_ALGORITHM:-NEW_GREEDY}
export HETU_SWITCH_PROFILE=${HETU_SWITCH_PROFILE:-INFO}
export HETU_INTERNAL_LOG_LEVEL=${HETU_INTERNAL_LOG_LEVEL:-WARN}
export HETU_MEMORY_PROFILE=${HETU_MEMORY_PROFILE:-WARN}
export PYTORCH_CUDA_ALLOC_CONF=${PYTORCH_CUDA_ALLOC_CONF:-expandable_segments:True}

echo "LLaMA-${MODEL_SIZE} on ${NUM_GPUS} GPUs, context ${SEQ_LEN}: buckets (${BUCKET_SIZES}), strategies (${STRATEGIES})"
if [ -n "${DRY_RUN:-}" ]; then exit 0; fi      # print the plan only
mkdir -p logs
python -m torch.distributed.run --nnodes=1 --nproc-per-node "${NUM_GPUS}" --master-addr 127.0.0.1 \
  --master-port "${MASTER_PORT}" -m hotspa_ae_b200.train.llama_hot_switch \
  --model_size "${MODEL_SIZE}" --hot_switch --reference_order --strategies "${STRATEGIES}" \
  --bucket_sizes "${BUCKET_SIZES}" --seq_length "${SEQ_LEN}" --vocab_size 30592 --zero --bf16 \
  --micro_batch_tokens 16384 --steps "${STEPS}" --epochs 1 --lr 1e-5 --adam_weight_decay 0.01 \
  --log_file "logs/hot_switch_${MODEL_SIZE}_${NUM_GPUS}gpus_${SEQ_LEN}.jsonl" ${DATA_ARGS} "${@:6}"
