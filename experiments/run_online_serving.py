#!/usr/bin/env python
"""Online (trace-driven) serving experiment, the counterpart of experiments/serving/run_online_test.sh: replays a trace
(`ts: .. prompt: .. shared: .. out: ..` lines, or a synthetic Poisson trace) through one prefill and one decode stage.

    python experiments/run_online_serving.py [--trace FILE] [--model tiny] [--requests 40] [--rate 200]

With one process both stages run as virtual ranks on one GPU.  Under torchrun with 2 x TP ranks, ranks below world/2
are the context stage (rank 0 reads the trace and shares each batch with its tensor-parallel group), the others
decode, and rank r hands its KV shard to rank r + world/2 -- the reference's layout (online_main.cc:117-170):

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 experiments/run_online_serving.py --model opt_6.7b

The report is the reference's: communication volume per batch (KV bytes, header bytes), send window, prefill time.
Both modes run on B200s: one process on one GPU, 1 + 1 processes on two GPUs, and 2 x TP 2 on four."""
import argparse
import json
import os
import queue
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--trace", default="")
    ap.add_argument("--model", default="tiny")
    ap.add_argument("--requests", type=int, default=40)
    ap.add_argument("--rate", type=float, default=200.0, help="synthetic arrivals per second")
    ap.add_argument("--input-len", type=int, default=512)
    ap.add_argument("--decode-steps", type=int, default=8)
    ap.add_argument("--decode-sleep-ms", type=float, default=0.0, help="stand-in for decoding, 25 in the reference")
    ap.add_argument("--device", default="cuda", choices=["cuda", "cpu"], help="cpu: host tensors and a host-memory heap (only under a model of "
                                                                              "the device entry points, as the tests run it)")
    ap.add_argument("--policy", default="fcfs", choices=["fcfs", "sjf", "aged"], help="order in which waiting requests are batched (fcfs: the reference)")
    ap.add_argument("--max-batch-tokens", type=int, default=0, help="limit on the active prompt tokens of one batch (0: none)")
    args = ap.parse_args()
    from fuselink_b200.models.llama import MODEL_ZOO, LlamaShard
    from fuselink_b200.parallel.symm import SymmetricHeap
    from fuselink_b200.serving.disagg import KVLink, ServeParams
    from fuselink_b200.serving.online import MAX_BATCH, OnlineDecode, OnlinePrefill, TraceReader, parse_trace
    cfg = MODEL_ZOO[args.model]
    p = ServeParams(cfg, MAX_BATCH, args.input_len, args.decode_steps)
    if args.trace:
        reqs = parse_trace(open(args.trace))
    else:
        from fuselink_b200.serving.tracegen import generate
        lines = generate(args.requests, args.rate, 32, args.input_len, 0.25, 4, 64, seed=0)
        reqs = parse_trace(lines)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1:
        return multi_process(args, cfg, p, reqs)
    net = LlamaShard(cfg, device=args.device, max_positions=args.input_len + args.decode_steps)
    pool = 2 * p.batch_size * p.max_blocks_per_req * cfg.layers * net.kvh_local * cfg.block_size * cfg.head_dim * 2
    heaps = SymmetricHeap.emulated(2, 2 * pool + (64 << 20))
    links = [[KVLink(h, p, net.kvh_local, name=f"kv{i}") for i in range(2)] for h in heaps]
    pre, dec = OnlinePrefill(p, net, links[0], 1), OnlineDecode(p, net, links[1], 0, sleep_ms=args.decode_sleep_ms)
    q = queue.Queue()
    TraceReader(reqs, q).start()
    from fuselink_b200.serving.scheduler import Scheduler
    sched = Scheduler(q, MAX_BATCH, p.input_len, policy=args.policy, max_batch_tokens=args.max_batch_tokens)
    finished, served = False, 0
    while not finished:
        batch, finished = sched.next_batch()
        if not batch:
            continue
        st = pre.serve_batch(batch)
        dec.serve_batch(args.decode_steps)
        served += len(batch)
        print(json.dumps({"batch": st.batch, "prompt_tokens": st.prompt_tokens, "kv_MB": st.kv_bytes / 1e6, "header_B": st.header_bytes,
                          "prefill_ms": round(st.prefill_ms, 3), "send_window_ms": round(st.send_ms, 3)}))
    print(json.dumps({"served": served, "batches": pre.batches, "total_kv_GB": sum(s.kv_bytes for s in pre.stats) / 1e9}))
    for h in heaps:
        h.close()


def multi_process(args, cfg, p, reqs):
    import threading

    import torch
    import torch.distributed as dist
    from fuselink_b200.models.llama import LlamaShard
    from fuselink_b200.parallel.symm import SymmetricHeap
    from fuselink_b200.serving.disagg import KVLink, ServeParams
    from fuselink_b200.serving.online import MAX_BATCH, OnlineDecode, OnlinePrefill, TraceReader
    rank, local, world = int(os.environ["RANK"]), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ["WORLD_SIZE"])
    assert world % 2 == 0, "half of the ranks prefill, half decode"
    cpu = args.device == "cpu"
    if cpu:
        dev = torch.device("cpu")
        dist.init_process_group("gloo")
    else:
        torch.cuda.set_device(local)
        dev = torch.device("cuda", local)
        dist.init_process_group("nccl", device_id=dev)
    tp = world // 2
    is_prefill = rank < tp
    groups = [dist.new_group(list(range(0, tp))), dist.new_group(list(range(tp, world)))]
    group = groups[0] if is_prefill else groups[1]
    p = ServeParams(cfg, MAX_BATCH, args.input_len, args.decode_steps, tp)
    net = LlamaShard(cfg, rank % tp, tp, group if tp > 1 else None, device=dev, max_positions=args.input_len + args.decode_steps)
    pool = 2 * p.batch_size * p.max_blocks_per_req * cfg.layers * net.kvh_local * cfg.block_size * cfg.head_dim * 2
    heap = SymmetricHeap.create(2 * pool + (64 << 20), device=-1 if cpu else local)
    links = [KVLink(heap, p, net.kvh_local, name=f"kv{i}") for i in range(2)]
    peer = rank + tp if is_prefill else rank - tp
    served = 0
    if is_prefill:
        pre = OnlinePrefill(p, net, links, peer)
        q = queue.Queue()
        if rank == 0:
            TraceReader(reqs, q).start()
        from fuselink_b200.serving.scheduler import Scheduler
        sched = Scheduler(q, MAX_BATCH, p.input_len, policy=args.policy, max_batch_tokens=args.max_batch_tokens)
        finished = False
        while not finished:
            box = [None]
            if rank == 0:
                batch, finished = sched.next_batch()
                box[0] = (batch, finished)
            if tp > 1:
                dist.broadcast_object_list(box, src=0, group=group)
            batch, finished = box[0]
            if not batch:
                continue
            st = pre.serve_batch(batch)
            served += len(batch)
            if rank == 0:
                print(json.dumps({"batch": st.batch, "prompt_tokens": st.prompt_tokens, "kv_MB": st.kv_bytes / 1e6, "header_B": st.header_bytes,
                                  "prefill_ms": round(st.prefill_ms, 3), "send_window_ms": round(st.send_ms, 3)}), flush=True)
        pre.send_end()
        heap.check_status("online prefill")
        if rank == 0:
            print(json.dumps({"served": served, "batches": pre.batches - 1, "total_kv_GB_per_rank": sum(s.kv_bytes for s in pre.stats) / 1e9}), flush=True)
    else:
        dec = OnlineDecode(p, net, links, peer, sleep_ms=args.decode_sleep_ms)
        while True:
            out = dec.serve_batch(args.decode_steps)
            if out["batch"] == 0:
                break
            served += out["batch"]
        heap.check_status("online decode")
        if rank == tp:
            print(json.dumps({"decoded_requests": served, "batches": dec.batches - 1}), flush=True)
    wd = threading.Timer(60.0, lambda: os._exit(0))      # the report is out: never hang in teardown
    wd.daemon = True
    wd.start()
    if not cpu:
        torch.cuda.synchronize()
    dist.barrier()
    heap.close()
    dist.destroy_process_group()
    wd.cancel()


if __name__ == "__main__":
    main()
