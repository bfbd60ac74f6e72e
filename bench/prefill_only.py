#!/usr/bin/env python
"""Prefill stage alone: one batch through a tensor-parallel shard group, timed with CUDA events (max over ranks).

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 bench/prefill_only.py --model opt_125m
    python bench/prefill_only.py --model tiny --device cpu        # functional check without a GPU
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
    ap.add_argument("--model", default="opt_125m")
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--input-len", type=int, default=1024)
    ap.add_argument("--block-size", type=int, default=32)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--device", default="cuda", choices=["cuda", "cpu"])
    args = ap.parse_args()
    from fuselink_b200.models.llama import MODEL_ZOO, LlamaShard
    import dataclasses
    rank, local, world = (int(os.environ.get(k, d)) for k, d in (("RANK", 0), ("LOCAL_RANK", 0), ("WORLD_SIZE", 1)))
    cpu = args.device == "cpu"
    if not cpu:
        torch.cuda.set_device(local)
    dev = torch.device("cpu") if cpu else torch.device("cuda", local)
    group = None
    if world > 1:
        dist.init_process_group("gloo" if cpu else "nccl", **({} if cpu else {"device_id": dev}))
        group = dist.group.WORLD
    cfg = dataclasses.replace(MODEL_ZOO[args.model], block_size=args.block_size)
    net = LlamaShard(cfg, rank, world, group, device=dev, dtype=torch.float32 if cpu else torch.bfloat16, max_positions=args.input_len)
    S = (args.input_len + cfg.block_size - 1) // cfg.block_size * cfg.block_size
    nblk = S // cfg.block_size
    pool = torch.zeros(args.batch * nblk * cfg.layers * net.kvh_local * cfg.block_size * cfg.head_dim, dtype=net.embed.dtype, device=dev)
    k_pool, v_pool = pool, torch.zeros_like(pool)
    table = torch.arange(args.batch * nblk, dtype=torch.int32, device=dev).view(args.batch, nblk)
    tokens = torch.randint(0, cfg.vocab, (args.batch, S), device=dev, generator=torch.Generator(device=dev).manual_seed(1))
    times = []
    for _ in range(args.iters):
        if cpu:
            t0 = time.perf_counter()
            net.prefill(tokens, k_pool, v_pool, table)
            times.append((time.perf_counter() - t0) * 1e3)
        else:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            e0.record()
            net.prefill(tokens, k_pool, v_pool, table)
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1))
    ms = torch.tensor([min(times[1:] or times)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    if rank == 0:
        print(json.dumps({"metric": "prefill only", "model": args.model, "tp": world, "batch": args.batch, "input_len": S,
                          "prefill_ms": float(ms.item()), "tokens_per_s": args.batch * S / (float(ms.item()) / 1e3)}), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
