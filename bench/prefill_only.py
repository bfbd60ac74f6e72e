#!/usr/bin/env python
"""Prefill stage alone: one batch through a tensor-parallel shard group, timed with CUDA events (max over ranks).  With
``--decode-steps N`` the same group then decodes N tokens greedily from the cache it has just filled and the latency per token
is reported too: the whole model on one tensor-parallel group without disaggregation, every sequence of the batch the same
length, which is what the reference's benchmark_tp2 / benchmark_tp4 jobs measure with SwiftTransformer's own benchmark
(experiments/serving/benchmark_tp2.sbatch:23-54).

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 bench/prefill_only.py --model opt_125m
    python -m torch.distributed.run --nproc-per-node 4 --master-addr 127.0.0.1 bench/prefill_only.py --model opt_13b --decode-steps 64
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
    ap.add_argument("--decode-steps", type=int, default=0, help="then decode this many tokens on the same group and report ms per token")
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
    net = LlamaShard(cfg, rank, world, group, device=dev, dtype=torch.float32 if cpu else torch.bfloat16,
                     max_positions=args.input_len + args.decode_steps + cfg.block_size)
    S = (args.input_len + cfg.block_size - 1) // cfg.block_size * cfg.block_size
    nblk = (S + args.decode_steps + cfg.block_size - 1) // cfg.block_size          # pages per sequence, decoded tokens included
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
    row = {"metric": "prefill only", "model": args.model, "tp": world, "batch": args.batch, "input_len": S,
           "prefill_ms": float(ms.item()), "tokens_per_s": args.batch * S / (float(ms.item()) / 1e3)}
    if args.decode_steps:
        # the prefill wrote pages as [block][layer][head][slot][dim]; the decoder reads [layer][block][slot][head][dim]
        first = net.prefill(tokens, k_pool, v_pool, table)
        nb, L, Hk, bs, D = args.batch * nblk, cfg.layers, net.kvh_local, cfg.block_size, cfg.head_dim
        kd = k_pool.view(nb, L, Hk, bs, D).permute(1, 0, 3, 2, 4).contiguous().view(-1)
        vd = v_pool.view(nb, L, Hk, bs, D).permute(1, 0, 3, 2, 4).contiguous().view(-1)
        cur = first
        if not cpu:
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
        t0 = time.perf_counter()
        for t in range(args.decode_steps):
            cur = net.decode_step(cur, torch.full((args.batch,), S + t, dtype=torch.long, device=dev), kd, vd, table, nb)
        if cpu:
            dms = (time.perf_counter() - t0) * 1e3
        else:
            e1.record()
            torch.cuda.synchronize()
            dms = e0.elapsed_time(e1)
        d = torch.tensor([dms], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(d, op=dist.ReduceOp.MAX)
        row.update({"metric": "prefill + decode on one group", "decode_steps": args.decode_steps,
                    "decode_ms_per_token": float(d.item()) / args.decode_steps,
                    "decode_tokens_per_s": args.batch * args.decode_steps / (float(d.item()) / 1e3)})
    if rank == 0:
        print(json.dumps(row), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
