#!/usr/bin/env bash
# Llama training under one static strategy on one node (the baseline the hot-switch runs are compared with;
# reference: hotspa/scripts/llama_static_parallel.sh).
#
#   bash llama_static_parallel.sh [MODEL_SIZE=7b] [SEQ_LEN=4096] [DP=2] [TP=2] [PP=2] [STEPS=50]
set -euo pipefail

MODEL_SIZE=${1:-7b}
SEQ_LEN=${2:-4096}
DP=${3:-2}
TP=${4:-2}
PP=${5:-2}
STEPS=${6:-50}
GLOBAL_BATCH_SIZE=${GLOBAL_BATCH_SIZE:-64}
MASTER_PORT=${MASTER_PORT:-29500}
NUM_GPUS=$(( DP * TP * PP ))

export HETU_INTERNAL_LOG_LEVEL=${HETU_INTERNAL_LOG_LEVEL:-WARN}
export HETU_MEMORY_PROFILE=${HETU_MEMORY_PROFILE:-WARN}
export PYTORCH_CUDA_ALLOC_CONF=${PYTORCH_CUDA_ALLOC_CONF:-expandable_segments:True}

echo "LLaMA-${MODEL_SIZE} static dp${DP} tp${TP} pp${PP} on ${NUM_GPUS} GPUs, sequences of ${SEQ_LEN}"
mkdir -p logs
python -m torch.distributed.run --nnodes=1 --nproc-per-node "${NUM_GPUS}" --master-addr 127.0.0.1 \
  --master-port "${MASTER_PORT}" -m hotspa_ae_b200.train.llama_static_parallel \
  --model_size "${MODEL_SIZE}" --dp "${DP}" --tp "${TP}" --pp "${PP}" --zero --bf16 \
  --seq_length "${SEQ_LEN}" --global_batch_size "${GLOBAL_BATCH_SIZE}" --fixed_len "${SEQ_LEN}" \
  --vocab_size 30592 --steps "${STEPS}" --lr 1e-5 \
  --log_file "logs/static_${MODEL_SIZE}_dp${DP}tp${TP}pp${PP}_${SEQ_LEN}.jsonl" "${@:7}"
