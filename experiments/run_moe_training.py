#!/usr/bin/env python
"""Expert-parallel MoE transformer training (the counterpart of the reference's Megatron-DeepSpeed experiment): every rank
holds num_experts / world experts of every layer, the rest of the model is replicated and its gradients are averaged.

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 experiments/run_moe_training.py --model mixtral_8x7b --layers 2
    python experiments/run_moe_training.py --model tiny_moe --device cpu --steps 5          # functional check without a GPU

Synthetic tokens, random-init weights; prints one JSON line per logging interval (loss, tokens/s over all ranks, timed on
the device and reduced as the maximum step time over ranks).  Has not been run on hardware yet (the MoE layer it is built
from has).  On several CPU ranks the run checks the plumbing only: the plain-PyTorch stand-in of the expert exchange carries
gradients for a rank's own tokens through its own experts, the fused CUDA path carries all of them.
"""
import argparse
import dataclasses
import json
import os
import sys
import threading
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="tiny_moe")
    ap.add_argument("--layers", type=int, default=0, help="override the number of layers (0: the model's own)")
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--log-every", type=int, default=5)
    ap.add_argument("--lr", type=float, default=0.01)
    ap.add_argument("--device", default="cuda", choices=["cuda", "cpu"])
    ap.add_argument("--shadow", type=int, default=0, help="replicate the N most favoured experts of every layer on every rank (CUDA, several ranks)")
    ap.add_argument("--reshadow-every", type=int, default=0, help="with --shadow: every K steps choose the shadowed experts of each layer "
                                                                  "again from the loads of the last batch")
    ap.add_argument("--reshadow-tolerance", type=float, default=0.15, help="copy slots stay empty once the busiest rank is within (1 + this) of the mean load")
    ap.add_argument("--host-heap", action="store_true", help="with --device cpu: build the symmetric heap in host memory and take the fused path "
                                                             "(only under a model of the device entry points, as the tests run it)")
    ap.add_argument("--checkpoint", default="", help="save the last state here (per rank: experts differ)")
    ap.add_argument("--resume", default="", help="load <path>.rank<r> written by --checkpoint (same world size) before training")
    a = ap.parse_args()
    from fuselink_b200.models.moe_transformer import MOE_ZOO, MoETransformer
    rank, local, world = (int(os.environ.get(k, d)) for k, d in (("RANK", 0), ("LOCAL_RANK", 0), ("WORLD_SIZE", 1)))
    cpu = a.device == "cpu"
    cfg = MOE_ZOO[a.model]
    if a.layers:
        cfg = dataclasses.replace(cfg, layers=a.layers)
    if a.shadow:
        cfg = dataclasses.replace(cfg, shadow_experts=a.shadow)
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
    fused = not cpu or a.host_heap
    if fused:
        from fuselink_b200.parallel.symm import SymmetricHeap
        T, k, H, F, E = a.batch * a.seq, cfg.topk, cfg.hidden, cfg.ffn, cfg.num_experts
        rows = (E // world + (a.shadow if world > 1 else 0)) * ((T * world + 127) // 128 * 128)
        per_layer = rows * H * 2 * 2 + 2 * T * k * H * 2 + rows * 4 + (1 << 20)        # the symmetric buffers of one MoE workspace
        if a.shadow and world > 1:                                                     # + expert weights and gradient staging of the copies
            per_layer += (E // world + 2 * a.shadow) * 3 * H * cfg.ffn * 2 + (1 << 20)
        heap = SymmetricHeap.create(cfg.layers * per_layer + (64 << 20), device=-1 if cpu else local)
    net = MoETransformer(cfg, a.batch * a.seq, heap, rank, world, device=dev, seed=0, fused_sgd_lr=a.lr if fused else 0.0)
    if a.resume:
        net.load_state_dict(torch.load(f"{a.resume}.rank{rank}", map_location=dev))
    params = net.dense_parameters() if fused else net.parameters()     # on the fused path the expert update is part of the wgrad GEMM
    opt = torch.optim.SGD(params, lr=a.lr)
    gen = torch.Generator(device=dev).manual_seed(100 + rank)
    t_mark, tok = time.perf_counter(), 0
    ev = None if cpu else (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
    if ev:
        ev[0].record()
    for step in range(1, a.steps + 1):
        tokens = torch.randint(0, cfg.vocab, (a.batch, a.seq), device=dev, generator=gen)
        labels = torch.roll(tokens, -1, 1)
        loss = net.train_step(tokens, labels, opt)
        tok += a.batch * a.seq
        if a.reshadow_every and step % a.reshadow_every == 0:
            for b in net.blocks:                 # between steps: nothing of the layer is in flight
                b.moe.reshadow(tolerance=a.reshadow_tolerance)
        if step % a.log_every == 0 or step == a.steps:
            if ev:
                ev[1].record()
                torch.cuda.synchronize()
                ms = ev[0].elapsed_time(ev[1])
                ev[0].record()
            else:
                ms = (time.perf_counter() - t_mark) * 1e3
                t_mark = time.perf_counter()
            t = torch.tensor([ms, float(loss)], dtype=torch.float64, device=dev)
            if world > 1:
                dist.all_reduce(t[:1], op=dist.ReduceOp.MAX)
                dist.all_reduce(t[1:], op=dist.ReduceOp.SUM)
                t[1] /= world
            if heap is not None:
                heap.check_status("training")
            if rank == 0:
                print(json.dumps({"step": step, "loss": round(float(t[1]), 4), "tokens_per_s": world * tok / (float(t[0]) / 1e3),
                                  "n_gpus": world, "model": a.model, "layers": cfg.layers}), flush=True)
            tok = 0
    if a.checkpoint:
        torch.save(net.state_dict(), f"{a.checkpoint}.rank{rank}")
    wd = threading.Timer(60.0, lambda: os._exit(0))
    wd.daemon = True
    wd.start()
    if world > 1:
        dist.barrier()
    if heap is not None:
        heap.close()
    if world > 1:
        dist.destroy_process_group()
    wd.cancel()


if __name__ == "__main__":
    main()
