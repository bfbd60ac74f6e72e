#!/usr/bin/env python
"""NCCL send/recv THROUGH the ncclNet plugin (the reference's bandwidth experiment, experiments/bw_test/
run_bw_test.sbatch:29-50: nccl-tests sendrecv_perf with NCCL_NET_PLUGIN=fuselink, 4 channels per peer, 512 KiB chunks).

Between machines NCCL uses its network transport by itself.  On one machine it prefers NVLink / shared memory, so this
script switches those off (NCCL_P2P_DISABLE=1, NCCL_SHM_DISABLE=1) to push the traffic of a rank pair through the
plugin; the number is then a test of the plugin under real NCCL, not a statement about NVLink.

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 bench/nccl_plugin_sendrecv.py
    ... --nnodes 2 ... bench/nccl_plugin_sendrecv.py --keep-intranode      # two machines: leave NCCL's transports alone

Every rank checks the received bytes and reads the plugin's own counters (selector decisions) from the library NCCL
loaded, so a run in which NCCL silently used another transport fails instead of reporting a number.
"""
import argparse
import ctypes
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
LIB_DIR = os.path.join(ROOT, "fuselink_b200", "lib")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--size-lo", type=int, default=20, help="log2 of the smallest message in bytes")
    ap.add_argument("--size-hi", type=int, default=30)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--keep-intranode", action="store_true", help="do not disable NCCL's P2P / SHM transports")
    args = ap.parse_args()
    # the environment NCCL reads at communicator creation; the values are the reference script's
    # NCCL looks the plugin up by name (libnccl-net-<name>.so) with dlopen.  Loading the library first by its full path makes
    # that lookup succeed whatever LD_LIBRARY_PATH was when the process started: the loader matches the soname.
    plugin_path = os.path.join(LIB_DIR, "libnccl-net-fuselink.so")
    preloaded = ctypes.CDLL(plugin_path, mode=ctypes.RTLD_GLOBAL)
    os.environ.setdefault("NCCL_NET_PLUGIN", "fuselink")
    os.environ.setdefault("NCCL_P2P_NET_CHUNKSIZE", "524288")
    os.environ.setdefault("NCCL_NCHANNELS_PER_NET_PEER", "4")
    os.environ.setdefault("NCCL_MIN_NCHANNELS", "4")
    os.environ.setdefault("NCCL_MAX_NCHANNELS", "4")
    os.environ.setdefault("NCCL_BUFFSIZE", "4194304")
    os.environ.setdefault("NCCL_NET_SHARED_BUFFERS", "0")
    os.environ.setdefault("NCCL_FUSELINK_DEGREE", "2")
    os.environ.setdefault("NCCL_FUSELINK_STEP", "1")
    os.environ.setdefault("NCCL_SOCKET_IFNAME", "lo" if not args.keep_intranode else os.environ.get("NCCL_SOCKET_IFNAME", ""))
    if not args.keep_intranode:
        os.environ["NCCL_P2P_DISABLE"] = "1"
        os.environ["NCCL_SHM_DISABLE"] = "1"
    import torch
    import torch.distributed as dist
    rank, local, world = int(os.environ["RANK"]), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ["WORLD_SIZE"])
    assert world % 2 == 0, "ranks are paired: r <-> r ^ 1"
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    peer = rank ^ 1
    results = []
    for lg in range(args.size_lo, args.size_hi + 1):
        n = (1 << lg) // 2
        src = torch.full((n,), float(rank + 1), dtype=torch.bfloat16, device=dev)
        dst = torch.zeros(n, dtype=torch.bfloat16, device=dev)

        def step():
            ops = [dist.P2POp(dist.isend, src, peer), dist.P2POp(dist.irecv, dst, peer)]
            for w in dist.batch_isend_irecv(ops):
                w.wait()

        for _ in range(args.warmup):
            step()
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.iters):
            step()
        e1.record()
        torch.cuda.synchronize()
        assert bool((dst == float(peer + 1)).all()), "received bytes differ"
        ms = torch.tensor([e0.elapsed_time(e1) / args.iters], device=dev, dtype=torch.float64)
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        results.append({"bytes": 1 << lg, "ms": float(ms.item()), "GBps_per_direction": (1 << lg) / (float(ms.item()) / 1e3) / 1e9})
    # did the traffic go through the plugin?  NCCL and this handle share one loaded library.
    lib = preloaded
    lib.fuselink_plugin_decisions.restype = ctypes.c_ulonglong
    used = torch.tensor([int(lib.fuselink_plugin_decisions())], device=dev)
    dist.all_reduce(used)
    if rank == 0:
        print(json.dumps({"metric": "NCCL send/recv through the FuseLink net plugin", "n_gpus": world, "plugin_selector_decisions": int(used.item()),
                          "results": results}), flush=True)
    ok = int(used.item()) > 0
    import threading
    wd = threading.Timer(60.0, lambda: os._exit(0 if ok else 4))
    wd.daemon = True
    wd.start()
    dist.barrier()
    dist.destroy_process_group()
    wd.cancel()
    if not ok:
        raise SystemExit("NCCL did not route any receive through the plugin")


if __name__ == "__main__":
    main()
