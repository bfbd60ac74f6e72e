#!/usr/bin/env python
"""Unbalanced p2p bandwidth sweep: GPU0 -> GPU1 (then 2 and 4 concurrent pairs), bf16 N(0,1), 1 KB .. 1 GB in
powers of two, 20 warm-up + 100 timed iterations, device-timed, max over the participating ranks.

Arms: this library's chunked put (ld/st and bulk-copy engines), the striped relay variant over idle GPUs
(--relays), and NCCL send/recv on the same box.  Every arm's last message is compared with its source after the timed
loop.  With --device-counters (default) the put kernel of the ld/st arm adds the bytes of every finished chunk to the
pinned host counters the monitor's sweeper reads; the total is printed beside the bytes sent.

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 bench/p2p_sweep.py [--pairs 1] [--size-hi 30]
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
    ap.add_argument("--pairs", type=int, default=1)
    ap.add_argument("--size-lo", type=int, default=10)
    ap.add_argument("--size-hi", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--iters", type=int, default=100)
    ap.add_argument("--relays", type=int, default=0, help="idle GPUs used as relays for the striped arm")
    ap.add_argument("--device-counters", type=int, default=1)
    ap.add_argument("--out", default="")
    args = ap.parse_args()
    rank = int(os.environ["RANK"]); local = int(os.environ["LOCAL_RANK"]); world = int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from fuselink_b200 import C
    from fuselink_b200.ops.comm import Channel, StripedP2P
    from fuselink_b200.parallel.selector import PathSelector
    from fuselink_b200.parallel.symm import SymmetricHeap, SymTensor
    assert 2 * args.pairs <= world
    maxb = 1 << args.size_hi
    heap = SymmetricHeap.create(2 * maxb + (512 << 20 if args.relays else 0) + (64 << 20), device=local)
    dstbuf = heap.alloc_tensor([maxb], torch.uint8)
    chans = {e: Channel(heap, f"p2p-{e}", engine=e) for e in ("ldst", "bulk")}
    striped = StripedP2P(heap, "sweep", 256 << 20) if args.relays else None
    mon = C.monitor_open("", True, world, 1, 160) if args.relays else None
    src = torch.randn(maxb // 2, device=dev, generator=torch.Generator(device=dev).manual_seed(777 + rank)).to(torch.bfloat16)
    sel = PathSelector(world) if args.device_counters else None
    ctr = chans["ldst"].attach_counters(sel) if sel is not None else None
    sent_ldst = 0
    # pair i: rank 2i -> rank 2i+1
    pair = rank // 2 if rank < 2 * args.pairs else -1
    sender = pair >= 0 and rank % 2 == 0
    receiver = pair >= 0 and rank % 2 == 1
    rows = []

    def timed(fn, nbytes):
        for _ in range(args.warmup):
            fn()
        dist.barrier(); torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / args.iters if pair >= 0 or args.relays else 0.0], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    for lg in range(args.size_lo, args.size_hi + 1):
        nbytes = 1 << lg
        row = {"bytes": nbytes}
        view = src.view(torch.uint8)[:nbytes]
        def check(what):
            """The message that arrived last equals its source (the sender's buffer is generated from a fixed seed)."""
            dist.barrier(); torch.cuda.synchronize()
            if receiver:
                want = torch.randn(maxb // 2, device=dev, generator=torch.Generator(device=dev).manual_seed(777 + rank - 1)).to(torch.bfloat16)
                assert torch.equal(dstbuf.local[:nbytes], want.view(torch.uint8)[:nbytes]), f"{what}: {nbytes} bytes arrived damaged"
                dstbuf.local[:nbytes].zero_()
            dist.barrier()

        for eng, ch in chans.items():
            def ours():
                # sender: one put launch; receiver: the wait for the arrival counter is part of the measured op
                if sender:
                    ch.put(view, rank + 1, dstbuf.offset, nbytes)
                elif receiver:
                    ch.expect(rank - 1, nbytes)
                    ch.wait([rank - 1])
            ms = timed(ours, nbytes)
            if eng == "ldst" and sender:
                sent_ldst += nbytes * (args.warmup + args.iters)
            check(f"fuselink {eng}")
            row[f"fuselink_{eng}_GBs"] = nbytes / ms / 1e6
            row[f"fuselink_{eng}_us"] = ms * 1e3

        def nccl():
            if sender:
                dist.send(view, rank + 1)
            elif receiver:
                dist.recv(dstbuf.local[:nbytes], rank - 1)
        ms = timed(nccl, nbytes)
        check("nccl")
        row["nccl_GBs"] = nbytes / ms / 1e6
        row["nccl_us"] = ms * 1e3
        if striped is not None and nbytes >= (8 << 20) and args.pairs == 1:
            idx = [0]
            # a message goes in pieces of at most (1 + relays) stripes of half a staging buffer each, issued back to back:
            # the relays' credits keep the source from overwriting a stripe that has not been forwarded yet
            piece = min(nbytes, (1 + args.relays) * striped.half_bytes)
            def relay():
                for off in range(0, nbytes, piece):
                    n = min(piece, nbytes - off)
                    stripes = C.select_paths(mon, 1 + args.relays, 1, 4 << 20, 512 * 1024, True, 0, 1, n, idx[0], C.monitor_now_ns())
                    for pth, _, _ in stripes[1:]:
                        C.monitor_release(mon, 0, pth)
                    idx[0] += 1
                    striped.transfer(0, 1, view[off:off + n] if rank == 0 else None,
                                     SymTensor(heap, dstbuf.offset + off, [n], torch.uint8), n, stripes)
            ms = timed(relay, nbytes)
            check("fuselink relay")
            row["fuselink_relay_GBs"] = nbytes / ms / 1e6
        heap.check_status("p2p sweep")
        if rank == 0:
            print(json.dumps(row), flush=True)
        rows.append(row)
    if ctr is not None:
        torch.cuda.synchronize()
        if rank == 0:
            print(json.dumps({"device_counter_bytes": int(ctr.sum()), "bytes_sent_by_the_ldst_arm": sent_ldst}), flush=True)
        sel.close()
    if rank == 0 and args.out:
        with open(args.out, "w") as f:
            json.dump({"pairs": args.pairs, "world": world, "rows": rows}, f, indent=1)
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
