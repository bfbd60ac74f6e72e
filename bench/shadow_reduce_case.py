"""One rank's share of the sum of replicated experts' weight gradients, timed on ONE GPU with the peers' buffers local:
the weight-gradient GEMM that deals its result rows out to ``world`` staging buffers, and the kernel that sums this rank's
blocks, applies the update and writes the rows into ``world`` copies.  On one GPU every store lands in local HBM, so the
numbers show what the kernels cost the SMs and the memory system, not the link.

    python bench/shadow_reduce_case.py --world 8 --groups 1 --rows 4096 --iters 5
"""
import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--world", type=int, default=8)
    ap.add_argument("--groups", type=int, default=1, help="replicated experts")
    ap.add_argument("--rows", type=int, default=4096, help="rows per expert on this rank (the contraction)")
    ap.add_argument("--M", type=int, default=28672)
    ap.add_argument("--N", type=int, default=4096)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--lr", type=float, default=0.01)
    a = ap.parse_args()
    from fuselink_b200.ops import gemm
    dev = torch.device("cuda", 0)
    W, G, M, N = a.world, a.groups, a.M, a.N
    cap = (a.rows + 127) // 128 * 128
    blk = gemm.push_block_log2(M, W)
    assert blk >= 0, "M must divide over the ranks"
    g = torch.Generator(device=dev).manual_seed(0)
    A = torch.randn(G * cap, M, generator=g, device=dev).to(torch.bfloat16)
    B = torch.randn(G * cap, N, generator=g, device=dev).to(torch.bfloat16)
    counts = torch.full((G,), a.rows, dtype=torch.int32, device=dev)
    # rank 0's view: its own staging receives from every source, the other ranks' stagings receive its rows
    stage = [torch.zeros(G, W, M // W, N, dtype=torch.bfloat16, device=dev) for _ in range(W)]
    copies = [torch.randn(G, M, N, generator=g, device=dev).to(torch.bfloat16) * 0.02 for _ in range(W)]
    status = torch.zeros(8, dtype=torch.int32, device=dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def timed(fn):
        for _ in range(a.warmup):
            fn()
        ts = []
        for _ in range(a.iters):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        return sorted(ts)[len(ts) // 2]

    t_push = timed(lambda: gemm.grouped_gemm_wgrad_push(A, B, counts, cap, G, [s.data_ptr() for s in stage], 0, blk, status=status))
    t_store = timed(lambda: gemm.grouped_gemm_wgrad(A, B, counts, cap, G, status=status))
    t_upd = timed(lambda: gemm.shadow_update(stage[0], copies[0], [c.data_ptr() for c in copies], G, 0, M, N, blk, M * N, a.lr))
    assert int(status[0]) == 0, status.tolist()
    flops = 2.0 * G * a.rows * M * N
    upd_bytes = G * (M // W) * N * 2 * (W + 1 + W)           # W partial rows and the own copy read, W copies written
    print(json.dumps({"world": W, "groups": G, "rows": a.rows, "M": M, "N": N,
                      "wgrad_push_ms": t_push, "wgrad_push_tflops": flops / t_push / 1e9,
                      "wgrad_store_ms": t_store, "wgrad_store_tflops": flops / t_store / 1e9,
                      "update_ms": t_upd, "update_bytes": upd_bytes, "update_GBs": upd_bytes / t_upd / 1e6,
                      "update_sent_GBs_if_remote": G * (M // W) * N * 2 * (W - 1) / t_upd / 1e6}))


if __name__ == "__main__":
    main()
