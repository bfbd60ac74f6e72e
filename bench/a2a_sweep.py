#!/usr/bin/env python
"""Uniform all-to-all bus bandwidth: per-pair 1 KB .. 128 MB at 2/4/8 GPUs, this library's one-launch push
all-to-all vs NCCL all_to_all_single; 20 warm-up + 100 timed iterations, device-timed, max over ranks.
busbw = per-rank bytes sent to OTHER ranks / time.

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 bench/a2a_sweep.py
"""
import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--size-lo", type=int, default=10)
    ap.add_argument("--size-hi", type=int, default=27)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--iters", type=int, default=100)
    ap.add_argument("--out", default="")
    args = ap.parse_args()
    rank = int(os.environ["RANK"]); local = int(os.environ["LOCAL_RANK"]); world = int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from fuselink_b200.ops.comm import Channel, all_to_all
    from fuselink_b200.parallel.symm import SymmetricHeap
    maxb = 1 << args.size_hi
    heap = SymmetricHeap.create(world * maxb + (64 << 20), device=local)
    recv = heap.alloc_tensor([world, maxb], torch.uint8)
    send = torch.randint(0, 255, (world, maxb), dtype=torch.uint8, device=dev)
    nccl_out = torch.empty(world * maxb, dtype=torch.uint8, device=dev)
    chans = {e: Channel(heap, f"a2a-{e}", engine=e) for e in ("ldst", "bulk")}
    rows = []

    def timed(fn):
        for _ in range(args.warmup):
            fn()
        dist.barrier(); torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / args.iters], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    from fuselink_b200.parallel.symm import SymTensor
    for lg in range(args.size_lo, args.size_hi + 1):
        per = 1 << lg
        row = {"per_pair_bytes": per, "world": world}
        s = send[:, :per].contiguous()
        rview = SymTensor(heap, recv.offset, (world, per), torch.uint8)
        for eng, ch in chans.items():
            ms = timed(lambda: all_to_all(ch, s, rview))
            row[f"fuselink_{eng}_busGBs"] = per * (world - 1) / ms / 1e6
            row[f"fuselink_{eng}_us"] = ms * 1e3
        flat = s.view(-1)
        out = nccl_out[: world * per]
        ms = timed(lambda: dist.all_to_all_single(out, flat))
        row["nccl_busGBs"] = per * (world - 1) / ms / 1e6
        row["nccl_us"] = ms * 1e3
        heap.check_status("a2a sweep")
        if lg == args.size_lo:
            assert torch.equal(rview.local.view(-1), out), "all-to-all result differs from NCCL"
        if rank == 0:
            print(json.dumps(row), flush=True)
        rows.append(row)
    if rank == 0 and args.out:
        with open(args.out, "w") as f:
            json.dump({"world": world, "rows": rows}, f, indent=1)
    import threading
    wd = threading.Timer(60.0, lambda: os._exit(0))
    wd.daemon = True
    wd.start()
    heap.close()
    dist.barrier()
    dist.destroy_process_group()
    wd.cancel()


if __name__ == "__main__":
    main()
