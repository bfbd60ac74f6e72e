#!/usr/bin/env python
"""Headline benchmark: MoE expert-parallel layer, forward + backward + SGD update, tokens/s.

Config (the MoE row of the baseline configs): hidden 4096, 8 experts (SwiGLU 4096 -> 14336 -> 4096), top-2
routing, 8192 tokens per GPU, bf16, Zipf(1.2) router bias, random-init N(0, 0.02) weights, synthetic
N(0, 1) activations.  Weak scaling: tokens per GPU fixed, the 8 experts are spread over the N GPUs.

    python bench.py --gpus 1 --steps 10 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29500 \
        bench.py --gpus 8 --steps 10 --warmup 3

Prints ONE JSON line on rank 0.  ``value`` is device-timed (CUDA events, max over ranks) with inputs resident
on the device; ``e2e`` is the same step driven through ``MoELayer`` with the host->device copy of each step's
activations from pinned memory and the device->host copy of every step's loss (into pinned memory; the host reads it once
the next step has been enqueued) inside the timed region.

On more than one GPU the layer evens out the skewed router's load by itself (``--shadow auto``): after the first warm-up
step it replicates the busiest experts where that is needed and spreads their rows over the ranks (``MoELayer.rebalance``);
the choice is fixed for the timed region and named in ``config.parallelism``.

After the fuselink arm the same process runs the stock PyTorch + NCCL formulation of the step (framework permute,
all_to_all_single, library grouped GEMM, autograd, torch.optim.SGD) with the same steps and warm-up -> ``vs_baseline``,
and the other parts of the headline metric (p2p and all-to-all bandwidth, DLRM samples/s), each beside its NCCL
counterpart -> ``other_metrics``.  ``--impl reference`` reports that the reference cannot be run here; ``--impl nccl``
runs the stock arm alone.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

REFERENCE_UNAVAILABLE = (
    "reference is not installable (no setup.py/pyproject; Makefile needs the absent nccl/ submodule sources) "
    "and its plugin refuses to initialise without RDMA verbs devices"
)


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.samples, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100", "-i", str(self.index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thr = threading.Thread(target=self._read, daemon=True)
            self.thr.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append((time.time(), line.strip()))

    def stop(self, t0: float, t1: float) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            pass
        rows = [s for t, s in self.samples if t0 <= t <= t1 + 0.1] or [s for _, s in self.samples[-3:]]
        sm, mx, reasons, power = [], [], set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in rows:
            p = [x.strip() for x in r.split(",")]
            if len(p) < 7:
                continue
            try:
                sm.append(float(p[0])); mx.append(float(p[1])); power.append(float(p[2]))
            except ValueError:
                continue
            for n, v in zip(names, p[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm), "power_w_max": max(power) if power else None}


class ResultLine:
    """Prints the result line exactly once: from the main thread when the run completes, or from a timer when what
    follows the device-timed region (the end-to-end region, the stock arm, the other metrics: a rank may raise there while
    the others wait in a collective) has not finished within its limit -- the line then carries what was complete by
    then plus a note, and the process ends with status 0 because the device-timed result is valid.  ``parts`` is filled
    in by the caller as the sections complete; ``make_line(parts)`` builds the line."""

    def __init__(self, rank: int, make_line, parts=None):
        self.rank, self.make_line = rank, make_line
        self.parts = parts if parts is not None else {}
        self.lock, self.printed, self.timer = threading.Lock(), False, None

    def emit(self) -> None:
        with self.lock:
            if self.printed:
                return
            self.printed = True
            if self.rank == 0:
                print(json.dumps(self.make_line(self.parts)))
            sys.stdout.flush()

    def arm(self, limit_s: float) -> None:
        def give_up():
            self.parts["unfinished"] = "a section after the device-timed region did not finish within its time limit"
            if self.parts.get("e2e") is None:
                self.parts["e2e"] = {"error": "the end-to-end region did not finish within its time limit"}
            self.emit()
            os._exit(0)

        self.timer = threading.Timer(limit_s, give_up)
        self.timer.daemon = True
        self.timer.start()

    def disarm(self) -> None:
        if self.timer is not None:
            self.timer.cancel()


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="fuselink", choices=["fuselink", "reference", "nccl"])
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--ffn", type=int, default=14336)
    ap.add_argument("--experts", type=int, default=8)
    ap.add_argument("--topk", type=int, default=2)
    ap.add_argument("--lr", type=float, default=0.01)
    ap.add_argument("--zipf", type=float, default=1.2)
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--device", default="cuda", choices=["cuda", "cpu"],
                    help="cpu: host tensors and a host-memory heap; only meaningful under a model of the device entry points (the tests run "
                         "the script that way to check its plumbing) and never a benchmark")
    ap.add_argument("--placement", default="balanced", choices=["balanced", "contiguous"],
                    help="which rank owns which expert (fuselink arm): balanced = evened out by the load the router's bias predicts "
                         "(no effect with one GPU or one expert per GPU); contiguous = expert e on rank e // (E / N)")
    ap.add_argument("--shadow", default="auto",
                    help="fuselink arm, N GPUs > 1.  auto (default): after the first warm-up step the layer looks at its own routing, "
                         "replicates as few of the busiest experts as it takes for no rank's own experts to exceed the mean load by more "
                         "than --tolerance, and splits the replicated experts' rows over the ranks so that every rank computes about the "
                         "mean (MoELayer.rebalance); the copies' weight gradients are summed over the ranks.  An integer N: the N experts "
                         "the router's bias favours most, their rows computed where they originate.  0: none")
    ap.add_argument("--shadow-slots", type=int, default=4, help="copy slots every rank reserves with --shadow auto (unused ones cost nothing per step)")
    ap.add_argument("--tolerance", type=float, default=0.05)
    ap.add_argument("--no-other", action="store_true", help="skip the p2p / all-to-all / DLRM numbers that follow the MoE arms")
    ap.add_argument("--no-baseline", action="store_true", help="skip the PyTorch + NCCL arm that follows the fuselink arm in the same process")
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp8"], help="fp8: block-scaled e4m3 (1x128) forward/dgrad GEMMs")
    return ap.parse_args()


def other_metrics(rank, world, local_rank, dev):
    """The rest of the headline metric -- p2p GB/s (GPU 0 -> GPU 1, 16 MiB and 1 GiB), all-to-all bus GB/s (128 MiB per
    pair) and DLRM samples/s (26 tables x 1M x 128 fp32, batch 65536, SGD) -- each beside its stock counterpart (NCCL
    send/recv, NCCL all_to_all_single, EmbeddingBag + NCCL all-to-all), measured in this process on the same GPUs:
    CUDA events, max over ranks, short loops.  The sweeps over every size are bench/p2p_sweep.py and bench/a2a_sweep.py."""
    import torch
    import torch.distributed as dist

    from fuselink_b200.ops.comm import Channel, all_to_all
    from fuselink_b200.parallel.symm import SymmetricHeap, SymTensor

    def timed(fn, warmup, iters):
        for _ in range(warmup):
            fn()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / iters], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    out = {}
    if world >= 2:
        big, per = 1 << 30, 128 << 20
        heap = SymmetricHeap.create(big + world * per + (64 << 20), device=local_rank)
        try:
            dst = heap.alloc_tensor([big], torch.uint8)
            src = torch.randint(0, 255, (big,), dtype=torch.uint8, device=dev)
            ch = Channel(heap, "bench-p2p", engine="bulk")
            p2p = {}
            for nbytes in (16 << 20, 1 << 30):
                def ours():
                    if rank == 0:
                        ch.put(src, 1, dst.offset, nbytes)
                    elif rank == 1:
                        ch.expect(0, nbytes)
                        ch.wait([0])

                def stock():
                    if rank == 0:
                        dist.send(src[:nbytes], 1)
                    elif rank == 1:
                        dist.recv(dst.local[:nbytes], 0)
                iters = 50 if nbytes < (1 << 28) else 15
                a, b = timed(ours, 5, iters), timed(stock, 5, iters)
                p2p[str(nbytes)] = {"fuselink_GBs": nbytes / a / 1e6, "nccl_GBs": nbytes / b / 1e6, "ratio": b / a}
            out["p2p_GBs"] = p2p
            recv = heap.alloc_tensor([world, per], torch.uint8)
            send = src[: world * per].view(world, per)
            ref = torch.empty(world * per, dtype=torch.uint8, device=dev)
            ca = Channel(heap, "bench-a2a", engine="bulk")
            a = timed(lambda: all_to_all(ca, send, recv), 3, 10)
            b = timed(lambda: dist.all_to_all_single(ref, send.view(-1)), 3, 10)
            same = bool(torch.equal(recv.local.view(-1), ref))
            out["a2a_busGBs"] = {"per_pair_bytes": per, "fuselink": per * (world - 1) / a / 1e6, "nccl": per * (world - 1) / b / 1e6,
                                 "ratio": b / a, "equal_to_nccl": same}
            heap.check_status("bench p2p / all-to-all")
            del dst, src, recv, send, ref
        finally:
            heap.close()
        torch.cuda.empty_cache()

    # DLRM, both arms
    from fuselink_b200.models.dlrm import DLRM, DLRMConfig, synthetic_batch
    from fuselink_b200.models.dlrm_baseline import BaselineDLRM
    torch.backends.cuda.matmul.allow_tf32 = True
    cfg = DLRMConfig()
    batches = [synthetic_batch(cfg, rank, world, dev, seed=s_) for s_ in range(2)]
    res = {}
    for arm in ("fuselink", "nccl"):
        heap = None
        if arm == "fuselink":
            bl = cfg.global_batch // world
            heap = SymmetricHeap.create(2 * bl * cfg.num_tables * cfg.dim * 4 + (16 << 20), device=local_rank)
            model = DLRM(cfg, heap, rank, world, device=dev)
        else:
            model = BaselineDLRM(cfg, rank, world, device=dev)
        opt = torch.optim.SGD(model.dense_parameters(), lr=cfg.lr)
        i = [0]

        def step():
            model.train_step(*batches[i[0] % 2], opt)
            i[0] += 1
        ms = timed(step, 3, 8)
        res[arm] = cfg.global_batch / (ms / 1e3)
        if heap is not None:
            heap.check_status("bench dlrm")
            heap.close()
        del model, opt
        torch.cuda.empty_cache()
    out["dlrm_samples_s"] = {"fuselink": res["fuselink"], "pytorch_nccl": res["nccl"], "ratio": res["fuselink"] / res["nccl"],
                             "config": "26 tables x 1M x 128 fp32 table-wise, pooling 20, Zipf(1.05), global batch 65536, SGD 0.01"}
    return out


def stock_arm(args, cfg, rank, world, dev, xs, fuselink_value):
    """The same step in its stock formulation (framework permute, NCCL all_to_all_single, library GEMMs, autograd,
    torch.optim.SGD; models/moe_baseline.py), timed like the fuselink arm: same inputs, steps and warm-up, CUDA events,
    max over ranks.  Experts sit where the in-order placement puts them: expert e on rank e // (E / N)."""
    import torch
    import torch.distributed as dist

    from fuselink_b200.models.moe_baseline import BaselineMoELayer

    import dataclasses
    layer = BaselineMoELayer(dataclasses.replace(cfg, fp8=False, shadow=(), placement=()), rank, world, device=dev, zipf_s=args.zipf, seed=0)
    opt = torch.optim.SGD([layer.router, layer.w13, layer.w2], lr=args.lr)

    def step(x):
        x = x.detach().requires_grad_(True)
        loss = layer(x).float().pow(2).mean()
        loss.backward()
        opt.step()
        opt.zero_grad(set_to_none=True)

    def sync_all():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(args.warmup):
        step(xs[i % len(xs)])
    sync_all()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        step(xs[i % len(xs)])
    e1.record()
    sync_all()
    tms = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(tms, op=dist.ReduceOp.MAX)
    ms = float(tms.item())
    value = world * cfg.tokens * args.steps / (ms / 1e3)
    gemm_used = layer.expert_gemm
    del layer, opt
    return {"impl": "pytorch+nccl: permute + all_to_all_single + library GEMMs + autograd + torch.optim.SGD, same process and inputs",
            "expert_gemm": gemm_used, "value": value, "unit": "tokens/s",
            "ms_per_step": ms / args.steps, "ratio": fuselink_value / value}


def main():
    args = parse()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": REFERENCE_UNAVAILABLE}))
        return 0

    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch multi-GPU runs with torch.distributed.run (one rank per GPU)")
    cpu = args.device == "cpu"
    if cpu:
        assert args.impl == "fuselink", "the host mode exists for the plumbing of the fuselink arm only"
        dev = torch.device("cpu")
        if world > 1:
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            dist.init_process_group("gloo", rank=rank, world_size=world)
    else:
        torch.cuda.set_device(local_rank)
        dev = torch.device("cuda", local_rank)
        if world > 1:
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from fuselink_b200.utils.timing import timing_event      # a CUDA timing event on a GPU, the host clock in the host mode

    from fuselink_b200.models.moe import MoELayer
    from fuselink_b200.ops.moe import MoEConfig

    cfg = MoEConfig(hidden=args.hidden, ffn=args.ffn, num_experts=args.experts, topk=args.topk, tokens=args.tokens,
                    fp8=args.dtype == "fp8" and args.impl == "fuselink")
    T, H = cfg.tokens, cfg.hidden

    if args.impl == "fuselink":
        from fuselink_b200.parallel.symm import SymmetricHeap

        W = world
        cap = (T * W + 127) // 128 * 128
        auto_shadow = args.shadow == "auto" and W > 1
        if auto_shadow:
            shadow = [-1] * min(args.shadow_slots, cfg.num_experts)     # empty copy slots, filled by rebalance() after warm-up step 1
        else:
            shadow = int(args.shadow) if (W > 1 and args.shadow != "auto") else 0
        rows = (cfg.num_experts // W + (len(shadow) if auto_shadow else shadow)) * cap
        heap_bytes = 2 * rows * H * 2 + rows * 4 + 2 * T * cfg.topk * H * 2 + (64 << 20)
        n_copy = len(shadow) if auto_shadow else shadow
        if n_copy:      # the expert weights and the staging of the copies' gradient rows live on the heap as well (MoEWorkspace.enable_push_reduce)
            heap_bytes += (cfg.num_experts // W + 2 * n_copy) * 3 * H * cfg.ffn * 2 + (1 << 20)
        heap = SymmetricHeap.create(heap_bytes, device=-1 if cpu else local_rank)
        layer = MoELayer(cfg, heap, rank, world, device=dev, zipf_s=args.zipf, seed=0, fused_sgd_lr=args.lr, shadow_experts=shadow,
                         placement=args.placement)
        expert_params = []          # updated inside the wgrad kernels' epilogue
    else:
        auto_shadow = False
        from fuselink_b200.models.moe_baseline import BaselineMoELayer

        heap = None
        layer = BaselineMoELayer(cfg, rank, world, device=dev, zipf_s=args.zipf, seed=0, placement=args.placement)
        expert_params = [layer.w13, layer.w2]
    opt = torch.optim.SGD([layer.router] + expert_params, lr=args.lr)

    gen = torch.Generator(device=dev).manual_seed(1234 + rank)
    n_inputs = 4
    xs = [torch.randn(T, H, generator=gen, device=dev).to(torch.bfloat16) for _ in range(n_inputs)]

    def step(x):
        x = x.detach().requires_grad_(True)
        out = layer(x)
        loss = out.float().pow(2).mean()
        loss.backward()
        opt.step()
        opt.zero_grad(set_to_none=True)
        return loss

    def sync_all():
        if world > 1:
            dist.barrier()
        if not cpu:
            torch.cuda.synchronize()

    def launches():
        return layer.ws.launches if getattr(layer, "ws", None) is not None else 0

    # ---------------------------------------------------------------- device-timed region
    for i in range(args.warmup):
        step(xs[i % n_inputs])
        if i == 0 and auto_shadow:
            sync_all()
            layer.rebalance(tolerance=args.tolerance)     # from the routing of the step just done; fixed from here on
    sync_all()
    if heap is not None:
        heap.check_status("warmup")
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.25)
    sync_all()
    l0 = launches()
    e0, e1 = timing_event(dev), timing_event(dev)
    t_wall0 = time.time()
    e0.record()
    for i in range(args.steps):
        step(xs[i % n_inputs])
    e1.record()
    sync_all()
    t_wall1 = time.time()
    ms = e0.elapsed_time(e1)
    n_launch = launches() - l0
    clocks = sampler.stop(t_wall0, t_wall1) if rank == 0 else None
    if heap is not None:
        heap.check_status("timed region")
    tms = torch.tensor([ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(tms, op=dist.ReduceOp.MAX)
    ms = float(tms.item())
    ms_per_step = ms / args.steps
    value = world * T * args.steps / (ms / 1e3)

    # ---------------------------------------------------------------- the result line
    shadowed = getattr(getattr(layer, "cfg", None), "shadow", ())
    placed = getattr(getattr(layer, "cfg", None), "placement", ())
    if args.impl == "nccl" and getattr(layer, "homes", None) is not None:
        placed = layer.homes.tolist()
    placed = list(placed) if placed and list(placed) != list(range(len(placed))) else None

    def make_line(parts):
        e2e, roof, base = parts.get("e2e"), parts.get("roofline"), parts.get("vs_baseline")
        flops_per_token = cfg.topk * 3 * 2 * cfg.hidden * cfg.ffn * 3       # 3 GEMM-equivalents, fwd + 2x bwd
        return {
            "metric": "MoE-EP tokens/s (fwd+bwd+SGD)", "value": value, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": base,
            "dtype": "fp8 e4m3 1x128 block-scaled (fwd, dgrad) + bf16 (wgrad)" if cfg.fp8 else "bf16", "data": "synthetic",
            "impl": args.impl,
            "config": {"model": "MoE-EP layer: hidden 4096, 8 experts SwiGLU 4096-14336-4096, top-2, Zipf(1.2) router bias"
                       if (args.hidden, args.ffn, args.experts, args.topk) == (4096, 14336, 8, 2) else
                       f"MoE-EP layer h{args.hidden} f{args.ffn} e{args.experts} k{args.topk}",
                       "global_batch": world * T, "seq_len": T, "tokens_per_gpu": T,
                       "parallelism": f"ep{world}" + (f", expert homes {placed}" if placed else "") + (f" + shadow experts {[e for e in shadowed if e >= 0]}" + (" chosen from the routing of warm-up step 1, their rows spread over the ranks' copies" if auto_shadow else "") if any(e >= 0 for e in shadowed) else ""),
                       "optimizer": "SGD lr %g (experts: fused into the wgrad epilogue)" % args.lr if args.impl == "fuselink" else "SGD lr %g" % args.lr,
                       "l2_policy": "per-step working set (expert weights + activations, > 1 GB) is larger than the 126 MB L2"},
            "tflops_per_gpu": flops_per_token * T * args.steps / (ms / 1e3) / 1e12,
            "clocks": clocks, "e2e": e2e, "gpu_launches": n_launch, "roofline": roof,
            **({"other_metrics": parts["other_metrics"]} if parts.get("other_metrics") is not None else {}),
            **({"unfinished": parts["unfinished"]} if "unfinished" in parts else {}),
            **({"host_mode": "device entry points modelled on the host: plumbing check, not a measurement"} if cpu else {}),
        }

    # The device-timed number exists from here on: whatever happens next, the line is printed exactly once.
    parts = {}
    result = ResultLine(rank, make_line, parts)
    result.arm(max(300.0, 60.0 * ms / 1e3))

    # ---------------------------------------------------------------- end-to-end region (public API)
    e2e = None
    if not args.no_e2e:
        try:
            host = [torch.randn(T, H).to(torch.bfloat16) for _ in range(2)]
            if cpu:
                def run_e2e(n):                                      # host mode: the copies in line, no streams
                    last, buf = 0.0, torch.empty(T, H, dtype=torch.bfloat16)
                    for i in range(n):
                        buf.copy_(host[i % 2])
                        last = float(step(buf).item())
                    return last
            else:
                host = [h.pin_memory() for h in host]
                # Input pipeline of the public API: each step's activations are copied from pinned host memory on a copy
                # stream into one of two device buffers while the previous step computes; the step waits for its own copy.
                copy_stream = torch.cuda.Stream(device=dev)
                dbufs = [torch.empty(T, H, dtype=torch.bfloat16, device=dev) for _ in range(2)]
                ready = [torch.cuda.Event() for _ in range(2)]
                consumed = [torch.cuda.Event() for _ in range(2)]

                def prefetch(i):
                    b = i % 2
                    with torch.cuda.stream(copy_stream):
                        copy_stream.wait_event(consumed[b])          # the step that last read this buffer has finished
                        dbufs[b].copy_(host[i % 2], non_blocking=True)
                        ready[b].record(copy_stream)

                # Device -> host: every step's loss is copied into pinned memory right behind the step and read by the host
                # once the NEXT step has been enqueued, so the GPU is never left without work while the host reads a number.
                loss_pinned = torch.zeros(2, dtype=torch.float32).pin_memory()
                loss_ready = [torch.cuda.Event() for _ in range(2)]

                def run_e2e(n):
                    last = 0.0
                    prefetch(0)
                    for i in range(n):
                        b = i % 2
                        torch.cuda.current_stream().wait_event(ready[b])
                        if i + 1 < n:
                            prefetch(i + 1)                          # next step's host -> device copy overlaps this step
                        loss = step(dbufs[b])
                        consumed[b].record()
                        loss_pinned[b:b + 1].copy_(loss.detach().reshape(1), non_blocking=True)   # this step's result, device -> host
                        loss_ready[b].record()
                        if i > 0:                                    # read the previous step's loss now that this step is queued
                            loss_ready[1 - b].synchronize()
                            last = float(loss_pinned[1 - b])
                    if n > 0:
                        loss_ready[(n - 1) % 2].synchronize()
                        last = float(loss_pinned[(n - 1) % 2])
                    return last

            run_e2e(2)
            sync_all()
            f0, f1 = timing_event(dev), timing_event(dev)
            f0.record()
            loss_host = run_e2e(args.steps)
            f1.record()
            sync_all()
            ems = torch.tensor([f0.elapsed_time(f1)], device=dev, dtype=torch.float64)
            if world > 1:
                dist.all_reduce(ems, op=dist.ReduceOp.MAX)
            parts["e2e"] = e2e = {"value": world * T * args.steps / (float(ems.item()) / 1e3), "unit": "tokens/s",
                   "h2d_bytes_per_step": T * H * 2, "d2h_bytes_per_step": 4, "last_loss": loss_host}
            if heap is not None:
                heap.check_status("e2e region")
        except Exception as e:  # noqa: BLE001 - the device-timed line above must still be reported
            parts["e2e"] = e2e = {"error": repr(e)}
            try:
                if not cpu:
                    torch.cuda.synchronize()
            except Exception:  # noqa: BLE001
                pass

    # ---------------------------------------------------------------- roofline of the fused path (hottest rank)
    roof = None
    try:
        if args.impl == "fuselink":
            from fuselink_b200.utils import roofline as rl
            rows = layer.ws.counts_now().sum().to(torch.float64).reshape(1)
            if world > 1:
                dist.all_reduce(rows, op=dist.ReduceOp.MAX)
            hot_rows = int(rows.item())
            m = rl.moe_step_model(T, world, cfg.hidden, cfg.ffn, cfg.topk, hot_rows, shadows=sum(1 for e in shadowed if e >= 0))
            roof = {"hot_rank_rows": hot_rows, "mean_rows": T * cfg.topk, "flops_hot_rank": m["flops"],
                    "nvlink_bytes_hot_rank": m["nvlink_bytes"], "target_ms": m["target_ms"],
                    "achieved_fraction": m["target_ms"] / ms_per_step, "peaks": rl.peaks().source,
                    "definition": "max(FLOPs / measured sustained cuBLAS bf16, NVLink bytes / 770 GB/s) on the rank with most routed rows"}
    except Exception as e:  # noqa: BLE001 - reporting only
        roof = {"error": repr(e)}
    parts["roofline"] = roof

    # ---------------------------------------------------------------- the stock arm, same process, same steps
    base = None
    if args.impl == "fuselink" and not args.no_baseline and not cpu:
        try:
            base = stock_arm(args, cfg, rank, world, dev, xs, value)
        except Exception as e:  # noqa: BLE001 - the fuselink numbers above must still be reported
            base = {"impl": "pytorch+nccl", "error": repr(e), "ratio": None}
    parts["vs_baseline"] = base

    # ---------------------------------------------------------------- the rest of the headline metric
    if args.impl == "fuselink" and not args.no_other and not cpu:
        layer = opt = None                       # the MoE arm's memory is not needed any more
        if heap is not None:
            heap.close()
            heap = None
        torch.cuda.empty_cache()
        try:
            parts["other_metrics"] = other_metrics(rank, world, local_rank, dev)
        except Exception as e:  # noqa: BLE001
            parts["other_metrics"] = {"error": repr(e)}

    result.disarm()
    result.emit()
    # the result is out: teardown must never be able to hang the job (a watchdog ends the process after 60 s)
    sys.stdout.flush()
    wd = threading.Timer(60.0, lambda: os._exit(0))
    wd.daemon = True
    wd.start()
    if heap is not None:
        heap.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    wd.cancel()
    return 0


if __name__ == "__main__":
    sys.exit(main())
