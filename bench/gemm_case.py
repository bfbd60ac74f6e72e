#!/usr/bin/env python
"""One grouped-GEMM case for timing and for ncu captures (small enough to end by itself under a profiler).

    python bench/gemm_case.py --case fwd1|fwd2|dact|dx|wgrad2|wgrad13 [--rows 8192] [--experts 1] [--iters 5]

Cases are the six GEMMs of one MoE expert step at hidden 4096 / ffn 14336 (per expert):
  fwd1   X[rows,4096]   x W13[28672,4096]^T   SWIGLU epilogue        fwd2   Act[rows,14336] x W2[4096,14336]^T  SCATTER
  dact   dY[rows,4096]  x W2[4096,14336]      DSWIGLU (B MN-major)   dx     dGU[rows,28672] x W13[28672,4096]   SCATTER (B MN-major)
  wgrad2 dY^T x Act -> [4096,14336]           WGRAD (K-grouped)      wgrad13 dGU^T x X -> [28672,4096]          WGRAD (K-grouped)
Prints device time (CUDA events, L2 flushed between iterations) and TFLOP/s against the measured cuBLAS peak.
"""
import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", default="fwd1")
    ap.add_argument("--rows", type=int, default=8192)
    ap.add_argument("--experts", type=int, default=1)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--ffn", type=int, default=14336)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--cublas", action="store_true", help="also time torch.matmul on the same shape")
    ap.add_argument("--group-m", type=int, default=16, help="row tiles that share a column of weight tiles in the tile order (L2 reuse)")
    ap.add_argument("--max-ctas", type=int, default=0, help="cap on the persistent grid (0: one CTA, or CTA pair, per SM)")
    ap.add_argument("--sgd", action="store_true", help="wgrad cases: apply W -= lr * dW in the epilogue (reads and rewrites the weights) as the MoE step does")
    ap.add_argument("--sweep", action="store_true", help="time the case for group-m 4/8/16/32 x both kernel variants, one JSON line each")
    args = ap.parse_args()
    from fuselink_b200.ops import gemm
    from fuselink_b200.utils import roofline
    from fuselink_b200.utils.timing import time_kernel
    G, cap, H, F = args.experts, args.rows, args.hidden, args.ffn
    dev = "cuda"
    bf = torch.bfloat16
    st = torch.zeros(8, dtype=torch.int32, device=dev)
    counts = torch.full((G,), cap, dtype=torch.int32, device=dev)

    def rnd(*shape, s=1.0):
        return (torch.randn(*shape, device=dev) * s).to(bf)

    info = torch.arange(G * cap, dtype=torch.int32, device=dev)
    sched = {"group_m": args.group_m, "max_ctas": args.max_ctas}           # read by the lambdas at call time
    if args.case == "fwd1":
        a, b = rnd(G * cap, H), rnd(G, 2 * F, H, s=0.02)
        out, gu = torch.empty(G * cap, F, dtype=bf, device=dev), torch.empty(G * cap, 2 * F, dtype=bf, device=dev)
        fn = lambda: gemm.grouped_gemm_rows(a, b, counts, cap, epilogue=gemm.EPI_SWIGLU, out=out, gu=gu, zero_tail=True, status=st, **sched)
        M, N, K = G * cap, 2 * F, H
    elif args.case == "fwd2":
        a, b = rnd(G * cap, F), rnd(G, H, F, s=0.02)
        dst = torch.empty(G * cap, H, dtype=bf, device=dev)
        fn = lambda: gemm.grouped_gemm_rows(a, b, counts, cap, epilogue=gemm.EPI_SCATTER, row_info=info, peers=[dst.data_ptr()], ldc=H, status=st, **sched)
        M, N, K = G * cap, H, F
    elif args.case == "dact":
        a, b = rnd(G * cap, H), rnd(G, H, F, s=0.02)
        gu, dgu = rnd(G * cap, 2 * F), torch.empty(G * cap, 2 * F, dtype=bf, device=dev)
        fn = lambda: gemm.grouped_gemm_rows(a, b, counts, cap, b_mn_major=True, epilogue=gemm.EPI_DSWIGLU, gu=gu, dgu=dgu, zero_tail=True, status=st, **sched)
        M, N, K = G * cap, F, H
    elif args.case == "dx":
        a, b = rnd(G * cap, 2 * F), rnd(G, 2 * F, H, s=0.02)
        dst = torch.empty(G * cap, H, dtype=bf, device=dev)
        fn = lambda: gemm.grouped_gemm_rows(a, b, counts, cap, b_mn_major=True, epilogue=gemm.EPI_SCATTER, row_info=info, peers=[dst.data_ptr()], ldc=H, status=st, **sched)
        M, N, K = G * cap, H, 2 * F
    elif args.case == "wgrad2":
        a, b = rnd(G * cap, H), rnd(G * cap, F)
        out = torch.zeros(G, H, F, dtype=bf, device=dev)
        fn = lambda: gemm.grouped_gemm_wgrad(a, b, counts, cap, G, out=out, sgd_lr=1e-6 if args.sgd else 0.0, status=st, **sched)
        M, N, K = H * G, F, cap
    elif args.case == "wgrad13":
        a, b = rnd(G * cap, 2 * F), rnd(G * cap, H)
        out = torch.zeros(G, 2 * F, H, dtype=bf, device=dev)
        fn = lambda: gemm.grouped_gemm_wgrad(a, b, counts, cap, G, out=out, sgd_lr=1e-6 if args.sgd else 0.0, status=st, **sched)
        M, N, K = 2 * F * G, H, cap
    else:
        raise SystemExit("unknown case")
    flops = 2.0 * M * N * K
    if args.sweep:
        from fuselink_b200._ext import require_native
        C = require_native()
        for pair in (0, 1, 2):
            C.gemm_set_variant(pair)
            for gm in (4, 8, 16, 32):
                sched["group_m"] = gm
                ms = time_kernel(fn, warmup=args.warmup, iters=args.iters)
                assert st[0].item() == 0, st.tolist()
                print(json.dumps({"case": args.case, "M": M, "N": N, "K": K, "pair": pair, "group_m": gm, "ms": ms, "tflops": flops / ms / 1e9,
                                  "frac_of_measured_cublas_burst": roofline.gemm_fraction(flops, ms)}))
        return
    ms = time_kernel(fn, warmup=args.warmup, iters=args.iters)
    assert st[0].item() == 0, st.tolist()
    row = {"case": args.case, "M": M, "N": N, "K": K, "ms": ms, "tflops": flops / ms / 1e9, "group_m": args.group_m,
           "frac_of_measured_cublas_burst": roofline.gemm_fraction(flops, ms), "peaks": roofline.peaks().source}
    if args.cublas:
        x, w = rnd(M, K), rnd(N, K)
        cms = time_kernel(lambda: x @ w.t(), warmup=args.warmup, iters=args.iters)
        row["cublas_ms"], row["cublas_tflops"] = cms, flops / cms / 1e9
    print(json.dumps(row))


if __name__ == "__main__":
    main()
