#!/usr/bin/env bash
# Small-scale evaluation in the shape of the reference's artifact run (hotspa/scripts/exprs_for_A100_40G.sh):
# LLaMA-3B on 8 GPUs, context lengths 4K / 8K / 16K / 32K, 10 steps each, hot switching against the best static
# strategy of that context length.  Step times land in logs/*.jsonl.
set -euo pipefail
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
STEPS=${STEPS:-10}
for SEQ_LEN in 4096 8192 16384 32768; do
  bash "${HERE}/llama_hot_switch.sh" 3b "${SEQ_LEN}" 8 "${STEPS}" synthetic
done
bash "${HERE}/llama_static_parallel.sh" 3b 4096 8 1 1 "${STEPS}"
bash "${HERE}/llama_static_parallel.sh" 3b 8192 2 2 2 "${STEPS}"
bash "${HERE}/llama_static_parallel.sh" 3b 16384 2 2 2 "${STEPS}"
bash "${HERE}/llama_static_parallel.sh" 3b 32768 1 4 2 "${STEPS}"
