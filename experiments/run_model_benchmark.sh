#!/usr/bin/env bash
# The whole model on ONE tensor-parallel group, no disaggregation: prefill of a batch whose sequences all have the same
# length, then a few greedy decoding steps, latency of both.  The reference runs SwiftTransformer's own benchmark this way
# (experiments/serving/benchmark_tp2.sbatch:23-54 and benchmark_tp4.sbatch: opt_30b, fp16, input 2048, block 32, batch 2).
#
#   TP=2 experiments/run_model_benchmark.sh                 # TP=4 for the other script
#   MODEL=llama2_7b INPUT_LEN=1024 TP=1 experiments/run_model_benchmark.sh
#   DEVICE=cpu MODEL=tiny INPUT_LEN=64 TP=2 experiments/run_model_benchmark.sh     # functional check without a GPU
set -euo pipefail
cd "$(dirname "$0")/.."
TP=${TP:-2}; MODEL=${MODEL:-opt_30b}; BATCH=${BATCH:-2}; INPUT_LEN=${INPUT_LEN:-2048}; BLOCK=${BLOCK:-32}
DECODE_STEPS=${DECODE_STEPS:-1}; DEVICE=${DEVICE:-cuda}; PORT=${PORT:-29671}
args=(bench/prefill_only.py --model "$MODEL" --batch "$BATCH" --input-len "$INPUT_LEN" --block-size "$BLOCK"
      --decode-steps "$DECODE_STEPS" --device "$DEVICE")
if [ "$TP" -gt 1 ]; then
  python -m torch.distributed.run --nnodes=1 --nproc-per-node "$TP" --master-addr 127.0.0.1 --master-port "$PORT" "${args[@]}"
else
  python "${args[@]}"
fi
