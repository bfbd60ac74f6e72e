#!/usr/bin/env bash
# Runs every measurement this repository reports, on NGPU GPUs of one machine, and appends one JSON line per result to
# OUT (default bench_results.jsonl).  Each multi-GPU command is a torchrun launch on 127.0.0.1; every number is timed on
# the device and reduced as the maximum over ranks by the script that prints it.
#
#   NGPU=1 bench/reproduce.sh            # kernels + flagship step on one GPU
#   NGPU=8 bench/reproduce.sh            # adds p2p / all-to-all sweeps, DLRM, serving and the NCCL arms
#   SECTIONS="moe dlrm" NGPU=8 bench/reproduce.sh
#   SECTIONS="moe-shadow shadow-reduce gemm-sweep monitor" NGPU=8 bench/reproduce.sh     # optional sections
set -uo pipefail
cd "$(dirname "$0")/.."
NGPU=${NGPU:-1}; OUT=${OUT:-bench_results.jsonl}; STEPS=${STEPS:-20}; WARMUP=${WARMUP:-5}
SECTIONS=${SECTIONS:-"gemm moe p2p a2a dlrm serving"}
PORT=29500
run() {  # label, command...
  local label=$1; shift
  echo "== $label" >&2
  if out=$("$@" 2> >(tail -n 5 >&2)); then echo "$out" | grep '^{' | sed "s/^{/{\"section\": \"$label\", /" >> "$OUT"; else echo "   failed: $label" >&2; fi
}
tr() { PORT=$((PORT + 1)); python -m torch.distributed.run --nnodes=1 --nproc-per-node "$NGPU" --master-addr 127.0.0.1 --master-port "$PORT" "$@"; }
launch() { if [ "$NGPU" -gt 1 ]; then tr "$@"; else python "$@"; fi; }

for s in $SECTIONS; do
  case $s in
    gemm)    # isolated grouped GEMMs of the flagship shape, the three tilings
      for v in 0 1 2; do FUSELINK_GEMM_PAIR=$v run "gemm variant=$v" python bench/gemm_case.py --case fwd1 --rows 8192 --iters 10; done ;;
    moe)
      for impl in fuselink nccl; do run "moe $impl" launch bench.py --impl "$impl" --gpus "$NGPU" --steps "$STEPS" --warmup "$WARMUP"; done ;;
    moe-shadow)   # not in the default list: what the default (--shadow auto: chosen and spread by rebalance()) is compared with
      if [ "$NGPU" -ge 2 ]; then
        run "moe contiguous placement, no shadows" tr bench.py --gpus "$NGPU" --steps "$STEPS" --warmup "$WARMUP" --placement contiguous --shadow 0 --no-baseline --no-other
        for n in 0 1 2 3; do run "moe shadow=$n (rows stay local)" tr bench.py --gpus "$NGPU" --steps "$STEPS" --warmup "$WARMUP" --shadow "$n" --no-baseline --no-other; done
      fi ;;
    monitor)   # not in the default list (no GPU needed): latency of a selector decision and of the table's calls
      for t in 1 4; do run "monitor decisions, $t thread(s)" fuselink_b200/lib/fuselink-monitor --bench 2000000 --threads "$t" --groups 8; done ;;
    shadow-reduce)   # not in the default list: the sum of the copies' gradients, own kernels against the all-reduce, and the two kernels alone
      run "push GEMM + update kernel, one GPU" python bench/shadow_reduce_case.py --world 8 --groups 1 --rows 4096 --iters 5
      if [ "$NGPU" -ge 2 ]; then
        for p in 1 0; do FUSELINK_PUSH_REDUCE=$p run "moe shadows forced, push=$p" tr bench.py --gpus "$NGPU" --steps "$STEPS" --warmup "$WARMUP" --tolerance 0 --no-baseline --no-other; done
      fi ;;
    gemm-sweep)   # not in the default list: tile order x kernel variant for every GEMM of the step
      for c in fwd1 fwd2 dact dx wgrad2 wgrad13; do run "gemm sweep $c" python bench/gemm_case.py --case "$c" --rows 16384 --iters 5 --sweep; done ;;
    p2p)
      if [ "$NGPU" -ge 2 ]; then run "p2p" tr bench/p2p_sweep.py --pairs 1; fi
      if [ "$NGPU" -ge 4 ]; then run "p2p 2 pairs" tr bench/p2p_sweep.py --pairs 2; run "p2p relays" tr bench/p2p_sweep.py --pairs 1 --relays 2; fi
      if [ "$NGPU" -ge 8 ]; then run "p2p 4 pairs" tr bench/p2p_sweep.py --pairs 4; fi ;;
    a2a)
      if [ "$NGPU" -ge 2 ]; then run "a2a" tr bench/a2a_sweep.py; fi ;;
    dlrm)
      for impl in fuselink nccl; do run "dlrm $impl" launch bench/dlrm_bench.py --impl "$impl" --steps "$STEPS" --warmup "$WARMUP"; done ;;
    serving)
      if [ "$NGPU" -ge 2 ]; then for kv in fuselink nccl; do run "serving $kv" tr bench/serving_bench.py --kv "$kv"; done
      else run "serving emulated" python bench/serving_bench.py --model tiny --emulate; fi ;;
  esac
done
echo "results in $OUT" >&2
