#!/usr/bin/env python
"""Single-GPU cases of the data-movement kernels, for timing and for ncu captures (each ends in seconds).

    python bench/kernel_case.py --case copy-ldst|copy-bulk|embbag-fwd|embbag-bwd|kvpack|dispatch|combine [--iters 3]

All "peer" buffers are regions of the same GPU (emulated symmetric heap), so the numbers are HBM-bound versions
of the kernels: bytes moved / time is compared with the measured device-copy bandwidth."""
import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", default="copy-ldst")
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=1)
    args = ap.parse_args()
    from fuselink_b200 import C
    from fuselink_b200.parallel.symm import SymmetricHeap
    from fuselink_b200.utils import roofline
    from fuselink_b200.utils.timing import time_kernel
    dev = "cuda"
    case = args.case
    if case.startswith("copy"):
        from fuselink_b200.ops.comm import Channel
        heaps = SymmetricHeap.emulated(2, (512 << 20) + (64 << 20))
        n = 256 << 20
        dst = [h.alloc_tensor([n], torch.uint8) for h in heaps]
        ch = Channel(heaps[0], "c", engine=case.split("-")[1])
        src = torch.randint(0, 255, (n,), dtype=torch.uint8, device=dev)
        fn = lambda: ch.put(src, 1, dst[0].offset)
        nbytes = 2 * n
    elif case.startswith("embbag"):
        from fuselink_b200.models.dlrm import DLRM, DLRMConfig, synthetic_batch
        cfg = DLRMConfig(num_tables=4, rows=1_000_000, global_batch=16384)
        heaps = SymmetricHeap.emulated(1, 2 * 16384 * 4 * 128 * 4 + (64 << 20))
        m = DLRM(cfg, heaps[0], 0, 1, device=dev)
        _, idx, _ = synthetic_batch(cfg, 0, 1, dev, seed=0)
        g = torch.randn(16384, 4, 128, device=dev)
        m.gpooled.local.copy_(g)
        if case == "embbag-fwd":
            fn = lambda: C.embbag(False, m.tables, idx, 0, 4, 16384, m.pooled.peers(), 0.0, 0, heaps[0].status_addr)
            nbytes = idx.numel() * 512 + idx.numel() * 8 + 16384 * 4 * 512
        else:
            fn = lambda: C.embbag(True, m.tables, idx, 0, 4, 16384, m.gpooled.peers(), 0.01, 0, heaps[0].status_addr)
            nbytes = 2 * idx.numel() * 512 + idx.numel() * 8 + 16384 * 4 * 512
    elif case == "kvpack":
        from fuselink_b200.models.llama import MODEL_ZOO
        from fuselink_b200.serving.disagg import KVLink, ServeParams
        cfg = MODEL_ZOO["llama3_8b"]
        p = ServeParams(cfg, batch_size=4, input_len=2048, num_decoding_step=0)
        heaps = SymmetricHeap.emulated(2, 2 * 4 * 128 * 32 * 8 * 16 * 128 * 2 + (64 << 20))
        links = [KVLink(h, p, 8) for h in heaps]
        nb = 4 * 128
        k = torch.randn(nb * 32 * 8 * 16 * 128, device=dev).to(torch.bfloat16)
        v = torch.randn_like(k)
        bt = torch.arange(nb, dtype=torch.int32, device=dev).view(4, 128)
        cnt = torch.full((4,), 128, dtype=torch.int32, device=dev)
        links[0].seq = 1
        fn = lambda: links[0].send_layers(1, k, v, nb, bt, bt.contiguous(), cnt, 0, 32)
        nbytes = 2 * 2 * k.numel() * 2
    elif case in ("dispatch", "combine"):
        from fuselink_b200.ops import moe as M
        cfg = M.MoEConfig()
        heaps = SymmetricHeap.emulated(1, 3 << 30)
        ws = M.MoEWorkspace(heaps[0], cfg)
        x = torch.randn(cfg.tokens, cfg.hidden, device=dev).to(torch.bfloat16)
        idx = torch.stack([torch.randperm(8, device=dev)[:2] for _ in range(cfg.tokens)]).int().contiguous()
        w = torch.rand(cfg.tokens, 2, device=dev)
        if case == "dispatch":
            def fn():
                ws.counts.local.zero_()
                M._dispatch(ws, x, idx, None, ws.xd, reuse=False)
            nbytes = cfg.tokens * cfg.hidden * 2 * 3
        else:
            out = torch.empty_like(x)
            fn = lambda: C.moe_combine(ws.comb.local, w, out, 2)
            nbytes = cfg.tokens * cfg.hidden * 2 * 3
    else:
        raise SystemExit("unknown case")
    ms = time_kernel(fn, warmup=args.warmup, iters=args.iters)
    for h in heaps:
        h.check_status(case)
    print(json.dumps({"case": case, "ms": ms, "bytes": nbytes, "GBs": nbytes / ms / 1e6, "frac_of_measured_copy": roofline.hbm_fraction(nbytes, ms)}))


if __name__ == "__main__":
    main()
