#!/usr/bin/env bash
# Bandwidth experiment, the counterpart of the reference's experiments/bw_test/run_bw_test.sbatch (nccl-tests
# sendrecv_perf through the plugin with 4 channels, 512 KiB chunks).  Two arms on one box:
#   1. device path: p2p sweep of this library vs NCCL over NVLink (needs >= 2 GPUs)
#   2. plugin path: the ncclNet plugin's TCP transport driven by two processes (no GPU needed)
#   3. NCCL through the plugin: torch.distributed send/recv with NCCL_NET_PLUGIN pointing at this build, NVLink and shared
#      memory switched off so that NCCL has to use its network transport (needs >= 2 GPUs; PLUGIN_ARM=1)
set -euo pipefail
cd "$(dirname "$0")/.."
export NCCL_P2P_NET_CHUNKSIZE=${NCCL_P2P_NET_CHUNKSIZE:-524288}
export NCCL_FUSELINK_DEGREE=${NCCL_FUSELINK_DEGREE:-2}
export NCCL_FUSELINK_STEP=${NCCL_FUSELINK_STEP:-1}
NGPU=${NGPU:-2}
if python -c "import torch,sys; sys.exit(0 if torch.cuda.device_count() >= $NGPU else 1)"; then
  python -m torch.distributed.run --nnodes=1 --nproc-per-node "$NGPU" --master-addr 127.0.0.1 bench/p2p_sweep.py --size-lo 10 --size-hi 30
fi
if [ "${PLUGIN_ARM:-0}" = 1 ]; then
  python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29631 bench/nccl_plugin_sendrecv.py --size-lo 20 --size-hi 28
fi
H=$(mktemp -u /tmp/fl_handle.XXXX)
LIB=fuselink_b200/lib
NCCL_SOCKET_IFNAME=${NCCL_SOCKET_IFNAME:-lo} $LIB/fl_net_harness $LIB/libnccl-net-fuselink.so recv "$H" --chunk 524288 --inflight 8 1073741824 &
NCCL_SOCKET_IFNAME=${NCCL_SOCKET_IFNAME:-lo} $LIB/fl_net_harness $LIB/libnccl-net-fuselink.so send "$H" --chunk 524288 --inflight 8 1073741824
wait
