#!/usr/bin/env bash
# Context (prefill) stage alone, tensor-parallel over TP_SZ GPUs (counterpart of experiments/serving/run_test_context.sh):
# times the prefill of one batch without a decode stage behind it.
set -euo pipefail
cd "$(dirname "$0")/.."
MODEL=${MODEL:-opt_125m}; BATCH=${BATCH:-1}; INPUT_LEN=${INPUT_LEN:-1024}; BLOCK=${BLOCK:-32}; TP_SZ=${TP_SZ:-2}
python -m torch.distributed.run --nnodes=1 --nproc-per-node "$TP_SZ" --master-addr 127.0.0.1 bench/prefill_only.py \
  --model "$MODEL" --batch "$BATCH" --input-len "$INPUT_LEN" --block-size "$BLOCK"
