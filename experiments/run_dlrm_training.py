#!/usr/bin/env python
"""DLRM training with table-wise sharded embeddings (the counterpart of the reference's DLRM experiment, the `herald`
submodule of .gitmodules:5-7): every rank owns some of the 26 tables, pools its tables for the whole global batch, the
pooled vectors travel to the samples' owners inside the embedding-bag kernel, the dense MLPs are data parallel.

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 experiments/run_dlrm_training.py
    python experiments/run_dlrm_training.py --device cpu --tables 5 --rows 300 --global-batch 64 --pooling 4 --steps 6   # no GPU

Synthetic Zipf-distributed indices and labels that depend on the inputs (so the loss can fall), random-init weights.
Prints one JSON line per logging interval: loss, samples/s over all ranks (device-timed on CUDA, maximum over ranks).
`--checkpoint PATH` writes PATH.rank<r> (each rank's tables differ); `--resume PATH` loads them at the same world size.
"""
import argparse
import json
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tables", type=int, default=26)
    ap.add_argument("--rows", type=int, default=1_000_000)
    ap.add_argument("--pooling", type=int, default=20)
    ap.add_argument("--global-batch", type=int, default=65536)
    ap.add_argument("--lr", type=float, default=0.01)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--log-every", type=int, default=10)
    ap.add_argument("--data-seeds", type=int, default=8, help="distinct synthetic batches, visited round robin")
    ap.add_argument("--device", default="cuda", choices=["cuda", "cpu"])
    ap.add_argument("--host-heap", action="store_true", help="with --device cpu: build the symmetric heap in host memory and take the fused path "
                                                             "(only under a model of the device entry points, as the tests run it)")
    ap.add_argument("--checkpoint", default="")
    ap.add_argument("--resume", default="")
    a = ap.parse_args()
    from fuselink_b200.models.dlrm import DLRM, DLRMConfig, synthetic_batch
    rank, local, world = (int(os.environ.get(k, d)) for k, d in (("RANK", 0), ("LOCAL_RANK", 0), ("WORLD_SIZE", 1)))
    cpu = a.device == "cpu"
    cfg = DLRMConfig(num_tables=a.tables, rows=a.rows, pooling=a.pooling, global_batch=a.global_batch, lr=a.lr)
    heap = None
    if cpu:
        dev = torch.device("cpu")
        if world > 1:
            dist.init_process_group("gloo")
    else:
        torch.cuda.set_device(local)
        dev = torch.device("cuda", local)
        if world > 1:
            dist.init_process_group("nccl", device_id=dev)
    if not cpu or a.host_heap:
        from fuselink_b200.parallel.symm import SymmetricHeap
        bl = cfg.global_batch // world
        heap = SymmetricHeap.create(2 * bl * cfg.num_tables * cfg.dim * 4 + (16 << 20), device=-1 if cpu else local)
    model = DLRM(cfg, heap, rank, world, device=dev)
    opt = torch.optim.SGD(model.dense_parameters(), lr=cfg.lr)
    start = 0
    if a.resume:
        ck = torch.load(f"{a.resume}.rank{rank}", map_location=dev)
        if ck["world"] != world:
            raise SystemExit(f"checkpoint was written by {ck['world']} ranks, this run has {world}")
        model.load_state_dict(ck["model"])
        opt.load_state_dict(ck["opt"])
        start = ck["step"]

    def batch(i):
        dense, idx, labels = synthetic_batch(cfg, rank, world, dev, seed=i % a.data_seeds)
        # a learnable target instead of coin flips: which side of zero the first dense feature is on
        return dense, idx, (dense[:, 0] > 0).to(labels.dtype).view_as(labels)

    def sync():
        if world > 1:
            dist.barrier()
        if not cpu:
            torch.cuda.synchronize()

    sync()
    t0, seen, loss = time.perf_counter(), 0, None
    ev = None if cpu else (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
    if ev:
        ev[0].record()
    for step in range(start, start + a.steps):
        d, i, l = batch(step)
        loss = model.train_step(d, i, l, opt)
        seen += 1
        if seen % a.log_every == 0 or step == start + a.steps - 1:
            if ev:
                ev[1].record()
            sync()
            sec = ev[0].elapsed_time(ev[1]) / 1e3 if ev else time.perf_counter() - t0
            t = torch.tensor([sec, float(loss)], dtype=torch.float64, device=dev)
            if world > 1:
                dist.all_reduce(t[:1], op=dist.ReduceOp.MAX)
                dist.all_reduce(t[1:], op=dist.ReduceOp.SUM)
                t[1] /= world
            if rank == 0:
                print(json.dumps({"step": step + 1, "loss": round(float(t[1]), 5), "samples_per_s": round(seen * cfg.global_batch / float(t[0]), 1),
                                  "world": world, "device": a.device}), flush=True)
            t0, seen = time.perf_counter(), 0
            if ev:
                ev[0].record()
    if heap is not None:
        heap.check_status("dlrm training")
    if a.checkpoint:
        torch.save({"model": model.state_dict(), "opt": opt.state_dict(), "step": start + a.steps, "world": world}, f"{a.checkpoint}.rank{rank}")
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
