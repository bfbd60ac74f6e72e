#!/usr/bin/env bash
# Offline disaggregated-serving experiment (counterpart of experiments/serving/run_test.sh): half of the GPUs prefill,
# half decode.  MODEL is a key of fuselink_b200.models.llama.MODEL_ZOO (opt_6.7b, opt_13b, opt_30b, llama2_7b, llama3_8b, ...).
set -euo pipefail
cd "$(dirname "$0")/.."
NGPU=${NGPU:-8}; MODEL=${MODEL:-llama3_8b}; INPUT_LEN=${INPUT_LEN:-2048}; BATCH=${BATCH:-16}; STEPS=${STEPS:-256}
for KV in fuselink nccl; do
  python -m torch.distributed.run --nnodes=1 --nproc-per-node "$NGPU" --master-addr 127.0.0.1 bench/serving_bench.py \
    --model "$MODEL" --kv "$KV" --batch "$BATCH" --input-len "$INPUT_LEN" --decode-steps "$STEPS"
done
