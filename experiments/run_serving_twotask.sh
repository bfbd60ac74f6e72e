#!/usr/bin/env bash
# Two serving jobs at the same time (counterpart of experiments/serving/run_test_twotask.sh, the contention scenario:
# two prefill->decode pairs with different prompt lengths whose KV hand-offs overlap).  Job 0 runs on GPUs 0,1 and
# job 1 on GPUs 2,3 (TP_SZ GPUs per stage each); both hand-offs cross the same NVSwitch at the same time.
set -euo pipefail
cd "$(dirname "$0")/.."
MODEL=${MODEL:-opt_6.7b}; BATCH=${BATCH:-1}; STEPS=${STEPS:-100}; BLOCK=${BLOCK:-32}; TP_SZ=${TP_SZ:-1}; KV=${KV:-fuselink}
INPUT_LEN_0=${INPUT_LEN_0:-1024}; INPUT_LEN_1=${INPUT_LEN_1:-512}
NP=$((2 * TP_SZ))
gpus() { local first=$1 n=$2 out=""; for ((i = 0; i < n; i++)); do out+="$((first + i)),"; done; echo "${out%,}"; }
run() {  # job index, first GPU, input length
  CUDA_VISIBLE_DEVICES=$(gpus "$2" "$NP") python -m torch.distributed.run --nnodes=1 --nproc-per-node "$NP" \
    --master-addr 127.0.0.1 --master-port $((29600 + $1)) -m fuselink_b200.serving \
    --model_name "$MODEL" --model_path dummy --precision bf16 --batch_size "$BATCH" --input_len "$3" \
    --block_size "$BLOCK" --num_decoding_step "$STEPS" --tp_size "$TP_SZ" --kv "$KV" | sed "s/^/[job $1] /"
}
run 0 0 "$INPUT_LEN_0" &
P0=$!
run 1 "$NP" "$INPUT_LEN_1" &
P1=$!
wait "$P0"; wait "$P1"
