#!/usr/bin/env python
"""Disaggregated serving: TTFT and decode tokens/s.

Llama-3-8B-shaped random-init bf16 model, half of the GPUs prefill and half decode (TP = world/2 inside each
stage), 16 prompts x 2048 tokens, 16-token pages, 256 greedy decode tokens.  KV moves prefill -> decode either
with the fused pack+send kernel, layer by layer while the prefill is still running (--kv fuselink), or as the
reference does it: whole K and V pools plus the small tensors in one NCCL group after the prefill (--kv nccl).

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 bench/serving_bench.py --kv fuselink
    python bench/serving_bench.py --model tiny --emulate        # both stages on one GPU (functional check only)
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
    ap.add_argument("--model", default="llama3_8b")
    ap.add_argument("--kv", default="fuselink", choices=["fuselink", "fuselink-nopipe", "nccl"])
    ap.add_argument("--batch", type=int, default=16)
    ap.add_argument("--input-len", type=int, default=2048)
    ap.add_argument("--decode-steps", type=int, default=256)
    ap.add_argument("--precision", default="bf16", choices=["bf16", "fp16", "fp32"], help="model and KV cache element type")
    ap.add_argument("--model-path", default="dummy", help="'dummy' = random weights, else a Hugging Face state_dict file or directory")
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--emulate", action="store_true")
    ap.add_argument("--device", default="cuda", choices=["cuda", "cpu"], help="cpu: host tensors and a host-memory heap (only under a model of "
                                                                              "the device entry points, as the tests run it)")
    args = ap.parse_args()
    from fuselink_b200.models.llama import MODEL_ZOO, LlamaShard, load_checkpoint_file
    from fuselink_b200.parallel.symm import SymmetricHeap
    from fuselink_b200.serving.disagg import DecodeStage, KVLink, PrefillStage, ServeParams, make_prompts

    rank = int(os.environ.get("RANK", 0)); local = int(os.environ.get("LOCAL_RANK", 0)); world = int(os.environ.get("WORLD_SIZE", 1))
    cpu = args.device == "cpu"
    if cpu:
        dev, heap_dev = torch.device("cpu"), -1
    else:
        torch.cuda.set_device(local)
        dev, heap_dev = torch.device("cuda", local), local

    def sync():
        if not cpu:
            torch.cuda.synchronize()

    cfg = MODEL_ZOO[args.model]
    dtype = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}[args.precision]
    if args.emulate or world == 1:
        p = ServeParams(cfg, args.batch, args.input_len, args.decode_steps, 1, dtype)
        net = LlamaShard(cfg, device=dev, dtype=dtype, max_positions=args.input_len + args.decode_steps)
        if args.model_path != "dummy":
            net.load_hf_state_dict(load_checkpoint_file(args.model_path))
        pool_bytes = 2 * p.batch_size * p.max_blocks_per_req * cfg.layers * net.kvh_local * cfg.block_size * cfg.head_dim * p.elem_bytes
        heaps = SymmetricHeap.emulated(2, pool_bytes + (64 << 20), device=max(heap_dev, 0))
        links = [KVLink(h, p, net.kvh_local) for h in heaps]
        pre = PrefillStage(p, net, links[0], 1, pipeline_layers=args.kv == "fuselink")
        dec = DecodeStage(p, net, links[1])
        prompts = make_prompts(p, dev)
        res = []
        for _ in range(args.iters):
            sync(); t0 = time.monotonic()
            rp = pre.run(prompts); rd = dec.run()
            res.append((rd.extra["t_first_token"] - t0, rp, rd))
        ttft, rp, rd = res[-1]
        print(json.dumps({"mode": "emulated-1gpu", "model": args.model, "ttft_ms": ttft * 1e3, "prefill_ms": rp.compute_ms,
                          "kv_ms": rp.kv_ms, "kv_GB": rp.kv_bytes / 1e9, "decode_tok_s": rd.tokens / (rd.compute_ms / 1e3)}))
        return
    assert world % 2 == 0
    if cpu:
        assert args.kv != "nccl", "the NCCL arm needs GPUs"
        dist.init_process_group("gloo")
    else:
        dist.init_process_group("nccl", device_id=dev)
    tp = world // 2
    is_prefill = rank < tp
    groups = [dist.new_group(list(range(0, tp))), dist.new_group(list(range(tp, world)))]
    tp_group = groups[0] if is_prefill else groups[1]
    tp_rank = rank % tp
    p = ServeParams(cfg, args.batch, args.input_len, args.decode_steps, tp, dtype)
    net = LlamaShard(cfg, tp_rank, tp, tp_group if tp > 1 else None, device=dev, dtype=dtype, max_positions=args.input_len + args.decode_steps)
    if args.model_path != "dummy":
        net.load_hf_state_dict(load_checkpoint_file(args.model_path))      # every shard cuts its part out of the full checkpoint
    pool_elems = p.batch_size * p.max_blocks_per_req * cfg.layers * net.kvh_local * cfg.block_size * cfg.head_dim
    heap = SymmetricHeap.create(2 * pool_elems * p.elem_bytes + (64 << 20), device=heap_dev)
    link = KVLink(heap, p, net.kvh_local)
    peer = rank + tp if is_prefill else rank - tp            # the reference's pairing: rank <-> rank + world/2
    prompts = make_prompts(p, dev)
    pre = PrefillStage(p, net, link, peer, pipeline_layers=args.kv == "fuselink") if is_prefill else None
    dec = DecodeStage(p, net, link, use_graph=True) if not is_prefill else None
    out = None
    for it in range(args.iters):
        dist.barrier(); sync()
        t0 = time.monotonic()
        if args.kv == "nccl":
            out = _nccl_iteration(p, net, link, pre, dec, prompts, peer, is_prefill, t0)
        elif is_prefill:
            rp = pre.run(prompts)
            out = {"prefill_ms": rp.compute_ms, "kv_ms": rp.kv_ms, "kv_GB": rp.kv_bytes / 1e9, "stage_ms": rp.elapsed_ms}
        else:
            rd = dec.run()
            out = {"ttft_ms": (rd.extra["t_first_token"] - t0) * 1e3, "decode_ms": rd.compute_ms, "wait_ms": rd.kv_ms,
                   "decode_tok_s": rd.tokens / (rd.compute_ms / 1e3)}
        heap.check_status("serving")
    gathered = [None] * world
    dist.all_gather_object(gathered, out)
    if rank == 0:
        pre_o, dec_o = gathered[:tp], gathered[tp:]
        line = {"metric": "disaggregated serving", "kv": args.kv, "model": args.model, "n_gpus": world, "tp": tp,
                "batch": p.batch_size, "input_len": p.input_len, "decode_steps": p.num_decoding_step,
                "ttft_ms": max(o["ttft_ms"] for o in dec_o), "decode_tok_s": min(o["decode_tok_s"] for o in dec_o),
                "prefill_ms": max(o["prefill_ms"] for o in pre_o), "kv_ms_max": max(o["kv_ms"] for o in pre_o),
                "kv_GB_per_rank": pre_o[0]["kv_GB"], "comm_over_elapsed": max(o["kv_ms"] for o in pre_o) / max(o["stage_ms"] for o in pre_o)}
        print(json.dumps(line), flush=True)
    # Teardown.  CUDA graphs that captured NCCL kernels are released before the process group goes away, and a
    # watchdog ends the process if the teardown stalls: the measurement is already printed.
    import threading
    wd = threading.Timer(60.0, lambda: os._exit(0))
    wd.daemon = True
    wd.start()
    if dec is not None:
        dec.graph = None
        dec.g_out = None
    sync()
    dist.barrier()
    heap.close()
    dist.destroy_process_group()
    wd.cancel()


def _nccl_iteration(p, net, link, pre, dec, prompts, peer, is_prefill, t0):
    """The reference's hand-off (model.hh:280-309): one group of 5 sends after the whole prefill -- first tokens, K pool,
    V pool, block table, block counts -- mirrored by 5 receives; the decoder then re-lays the pages out for its pool."""
    cfg = p.model
    B, cb, mb = p.batch_size, p.context_blocks_per_req, p.max_blocks_per_req
    dev = prompts.device
    kvh, bs, D, L = net.kvh_local, cfg.block_size, cfg.head_dim, cfg.layers
    n = B * cb * L * kvh * bs * D
    if is_prefill:
        e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        e0.record()
        first = net.prefill(prompts, pre.k_pool, pre.v_pool, pre.src_bt, None)
        e1.record()
        ops = [dist.P2POp(dist.isend, t, peer) for t in (first, pre.k_pool, pre.v_pool, pre.src_bt, pre.nblocks)]
        for r in dist.batch_isend_irecv(ops):
            r.wait()
        e2.record()
        torch.cuda.synchronize()
        return {"prefill_ms": e0.elapsed_time(e1), "kv_ms": e1.elapsed_time(e2), "kv_GB": 2 * n * p.elem_bytes / 1e9, "stage_ms": e0.elapsed_time(e2)}
    first = torch.empty(B, dtype=torch.long, device=dev)
    k_in = torch.empty(n, dtype=p.dtype, device=dev); v_in = torch.empty_like(k_in)
    bt = torch.empty(B, cb, dtype=torch.int32, device=dev); nb = torch.empty(B, dtype=torch.int32, device=dev)
    w0, w1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    w0.record()
    ops = [dist.P2POp(dist.irecv, t, peer) for t in (first, k_in, v_in, bt, nb)]
    for r in dist.batch_isend_irecv(ops):
        r.wait()
    # layout change into the decode pool: [blk][L][h][s][d] -> [L][blk'][s][h][d]
    kd = link.k_pool.local.view(L, link.pool_blocks, bs, kvh, D); vd = link.v_pool.local.view(L, link.pool_blocks, bs, kvh, D)
    dst_blocks = dec.bt[:, :cb].reshape(-1).long()
    kd[:, dst_blocks] = k_in.view(B * cb, L, kvh, bs, D).permute(1, 0, 3, 2, 4)
    vd[:, dst_blocks] = v_in.view(B * cb, L, kvh, bs, D).permute(1, 0, 3, 2, 4)
    w1.record()
    torch.cuda.synchronize()
    t_first = time.monotonic()
    gen, ms = dec.decode(first)              # same decode loop (CUDA graph) as the other arms
    return {"ttft_ms": (t_first - t0) * 1e3, "decode_ms": ms, "wait_ms": w0.elapsed_time(w1),
            "decode_tok_s": B * p.num_decoding_step / (ms / 1e3)}


if __name__ == "__main__":
    main()
