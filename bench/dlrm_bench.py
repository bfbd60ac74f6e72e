#!/usr/bin/env python
"""DLRM samples/s: 26 tables x 1M x 128 fp32 table-wise sharded, pooling 20, Zipf(1.05) indices, global batch
65536, SGD 0.01; fused embedding-bag + all-to-all kernels vs torch EmbeddingBag + NCCL all_to_all.

    python bench/dlrm_bench.py --impl fuselink|nccl [--steps 20 --warmup 5]
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 bench/dlrm_bench.py --impl fuselink

Device-timed with CUDA events, max over ranks; prints one JSON line on rank 0."""
import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist

torch.backends.cuda.matmul.allow_tf32 = True   # dense MLPs on the tensor cores (both arms)
torch.backends.cudnn.allow_tf32 = True


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--impl", default="fuselink", choices=["fuselink", "nccl"])
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--rows", type=int, default=1_000_000)
    ap.add_argument("--global-batch", type=int, default=65536)
    ap.add_argument("--tables", type=int, default=26)
    ap.add_argument("--device", default="cuda", choices=["cuda", "cpu"], help="cpu: plumbing check under a model of the device entry points (tests), "
                                                                              "never a measurement")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", 0)); local = int(os.environ.get("LOCAL_RANK", 0)); world = int(os.environ.get("WORLD_SIZE", 1))
    cpu = args.device == "cpu"
    if cpu:
        assert args.impl == "fuselink"
        dev = torch.device("cpu")
        if world > 1:
            dist.init_process_group("gloo")
    else:
        torch.cuda.set_device(local)
        dev = torch.device("cuda", local)
        if world > 1:
            dist.init_process_group("nccl", device_id=dev)
    from fuselink_b200.utils.timing import timing_event
    from fuselink_b200.models.dlrm import DLRM, DLRMConfig, synthetic_batch
    cfg = DLRMConfig(num_tables=args.tables, rows=args.rows, global_batch=args.global_batch)
    heap = None
    if args.impl == "fuselink":
        from fuselink_b200.parallel.symm import SymmetricHeap
        bl = cfg.global_batch // world
        heap = SymmetricHeap.create(2 * bl * cfg.num_tables * cfg.dim * 4 + (16 << 20), device=-1 if cpu else local)
        model = DLRM(cfg, heap, rank, world, device=dev)
        step_fn = model.train_step
    else:
        from fuselink_b200.models.dlrm_baseline import BaselineDLRM
        model = BaselineDLRM(cfg, rank, world, device=dev)
        step_fn = model.train_step
    opt = torch.optim.SGD(model.dense_parameters(), lr=cfg.lr)
    batches = [synthetic_batch(cfg, rank, world, dev, seed=s) for s in range(4)]

    def sync():
        if world > 1:
            dist.barrier()
        if not cpu:
            torch.cuda.synchronize()

    for i in range(args.warmup):
        step_fn(*batches[i % 4], opt)
    sync()
    e0, e1 = timing_event(dev), timing_event(dev)
    e0.record()
    for i in range(args.steps):
        loss = step_fn(*batches[i % 4], opt)
    e1.record()
    sync()
    ms = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    if heap is not None:
        heap.check_status("dlrm bench")
    ms = float(ms) / args.steps
    t_local = model.t_local
    gather_bytes = cfg.global_batch * cfg.pooling * t_local * cfg.dim * 4
    if rank == 0:
        print(json.dumps({"metric": "DLRM samples/s", "impl": args.impl, "value": cfg.global_batch / (ms / 1e3), "unit": "samples/s",
                          "n_gpus": world, "ms_per_step": ms, "loss": float(loss), "steps": args.steps, "warmup": args.warmup,
                          "config": {"tables": cfg.num_tables, "rows": cfg.rows, "dim": cfg.dim, "pooling": cfg.pooling,
                                     "global_batch": cfg.global_batch, "tables_on_rank0": t_local},
                          "rank0_gather_bytes_per_step": gather_bytes,
                          "gpu_launches_per_step": getattr(model, "launches", 0) / (args.steps + args.warmup)}))
    import threading
    wd = threading.Timer(60.0, lambda: os._exit(0))
    wd.daemon = True
    wd.start()
    if heap is not None:
        heap.close()
    if world > 1:
        dist.destroy_process_group()
    wd.cancel()


if __name__ == "__main__":
    main()
