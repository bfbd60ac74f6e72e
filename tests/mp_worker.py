"""Worker of tests/test_multigpu.py: one process per GPU (torchrun).  Checks, against NCCL / PyTorch results
computed in the same job, the symmetric heap, p2p put, all-to-all, the MoE expert-parallel step and the DLRM step."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist


def main():
    rank, local, world = int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from fuselink_b200.models.dlrm import DLRM, DLRMConfig, synthetic_batch
    from fuselink_b200.models.dlrm_baseline import BaselineDLRM
    from fuselink_b200.models.moe import MoELayer
    from fuselink_b200.models.moe_baseline import BaselineMoELayer
    from fuselink_b200.ops.comm import Channel, all_to_all, barrier
    from fuselink_b200.ops.moe import MoEConfig
    from fuselink_b200.parallel.symm import SymmetricHeap

    heap = SymmetricHeap.create(512 << 20, device=local)
    # ---- p2p ring: rank r -> r+1 -------------------------------------------------------------------------
    for engine in ("ldst", "bulk"):
        ch = Channel(heap, f"ring-{engine}", engine=engine)
        n = (3 << 20) + 48
        dst = heap.alloc_tensor([n], torch.uint8)
        src = torch.randint(0, 255, (n,), dtype=torch.uint8, device=dev, generator=torch.Generator(device=dev).manual_seed(rank))
        ch.put(src, (rank + 1) % world, dst.offset)
        ch.expect((rank - 1) % world, n)
        ch.wait([(rank - 1) % world])
        torch.cuda.synchronize()
        want = torch.randint(0, 255, (n,), dtype=torch.uint8, device=dev, generator=torch.Generator(device=dev).manual_seed((rank - 1) % world))
        assert torch.equal(dst.local, want), f"p2p {engine} mismatch on rank {rank}"
        # ---- all-to-all vs NCCL --------------------------------------------------------------------------
        per = 100_000
        send = torch.randn(world, per, device=dev)
        recv = heap.alloc_tensor([world, per], torch.float32)
        ref = torch.empty(world * per, device=dev)
        for _ in range(3):
            all_to_all(ch, send, recv)
            dist.all_to_all_single(ref, send.view(-1))
            torch.cuda.synchronize()
            assert torch.equal(recv.local.view(-1), ref), f"all-to-all {engine} mismatch on rank {rank}"
            barrier(heap, "a2a-reuse")          # the receive buffer is reused by the next iteration
    heap.check_status("comm")

    # ---- MoE: fused path vs the PyTorch + NCCL formulation, same weights, same inputs ----------------------
    cfg = MoEConfig(hidden=512, ffn=1024, num_experts=8, topk=2, tokens=768)
    fused = MoELayer(cfg, heap, rank, world, device=dev, seed=4, fused_sgd_lr=0.0)
    base = BaselineMoELayer(cfg, rank, world, device=dev, seed=4)
    for step in range(2):
        g = torch.Generator(device=dev).manual_seed(50 + step * 10 + rank)
        x = torch.randn(cfg.tokens, cfg.hidden, generator=g, device=dev).to(torch.bfloat16)
        xa, xb = x.clone().requires_grad_(True), x.clone().requires_grad_(True)
        oa, ob = fused(xa), base(xb)
        (oa.float().pow(2).mean()).backward()
        (ob.float().pow(2).mean()).backward()
        torch.cuda.synchronize()
        heap.check_status("moe")

        def close(a, b, what, tol=5e-2):
            err = (a.float() - b.float()).abs().max().item()
            den = b.float().abs().max().item() + 1e-6
            assert err < tol * den, f"rank {rank} step {step} {what}: err {err} vs {den}"

        close(oa, ob, "out")
        close(xa.grad, xb.grad, "dx")
        close(fused.router.grad, base.router.grad, "drouter", 8e-2)
        from fuselink_b200.ops import gemm
        dg, du = gemm.deinterleave_gate_up(fused.w13.grad)
        F = cfg.ffn
        close(dg, base.w13.grad[:, :F], "dWgate")
        close(du, base.w13.grad[:, F:], "dWup")
        close(fused.w2.grad, base.w2.grad, "dW2")
        for m in (fused, base):
            m.zero_grad(set_to_none=True)

    # ---- MoE with the two hottest experts replicated on every rank ---------------------------------------------
    if True:
        from fuselink_b200.ops import gemm
        sh = MoELayer(cfg, heap, rank, world, device=dev, seed=4, fused_sgd_lr=0.0, name="moe_sh", shadow_experts=2)
        epr, F = cfg.num_experts // world, cfg.ffn
        for step in range(2):
            g = torch.Generator(device=dev).manual_seed(90 + step * 10 + rank)
            x = torch.randn(cfg.tokens, cfg.hidden, generator=g, device=dev).to(torch.bfloat16)
            xa, xb = x.clone().requires_grad_(True), x.clone().requires_grad_(True)
            oa, ob = sh(xa), base(xb)
            (oa.float().pow(2).mean()).backward()
            (ob.float().pow(2).mean()).backward()
            torch.cuda.synchronize()
            heap.check_status("moe shadow")

            def close(a, b, what, tol=5e-2):
                err = (a.float() - b.float()).abs().max().item()
                den = b.float().abs().max().item() + 1e-6
                assert err < tol * den, f"rank {rank} step {step} shadow {what}: err {err} vs {den}"

            close(oa, ob, "out")
            close(xa.grad, xb.grad, "dx")
            dg, du = gemm.deinterleave_gate_up(sh.w13.grad)
            for le in range(epr):
                e = rank * epr + le
                slot = epr + sh.cfg.shadow.index(e) if e in sh.cfg.shadow else le     # the summed gradient sits in the copy
                close(dg[slot], base.w13.grad[le, :F], f"dWgate expert {e}")
                close(du[slot], base.w13.grad[le, F:], f"dWup expert {e}")
                close(sh.w2.grad[slot], base.w2.grad[le], f"dW2 expert {e}")
            for m in (sh, base):
                m.zero_grad(set_to_none=True)

    # ---- shadowed experts with the fused update: the copies' gradient rows are pushed by the weight-gradient GEMMs to the
    # rank that sums them, which writes the updated rows into every copy; against the all-reduce formulation ----------
    if world > 1:
        lr, arms = 0.01, {}
        for push in ("1", "0"):
            os.environ["FUSELINK_PUSH_REDUCE"] = push
            arms[push] = MoELayer(cfg, heap, rank, world, device=dev, seed=4, fused_sgd_lr=lr, name="moe_push" + push, shadow_experts=2)
        os.environ.pop("FUSELINK_PUSH_REDUCE")
        assert arms["1"].ws.push is not None and arms["0"].ws.push is None
        before = {n: getattr(arms["0"], n).detach().float().clone() for n in ("w13", "w2")}
        for step in range(3):
            g = torch.Generator(device=dev).manual_seed(170 + step * 10 + rank)
            x = torch.randn(cfg.tokens, cfg.hidden, generator=g, device=dev).to(torch.bfloat16)
            for m in arms.values():
                m(x.clone().requires_grad_(True)).float().pow(2).sum().backward()
            torch.cuda.synchronize()
            heap.check_status("moe push")
        arms["1"].weights_ready()           # the peers write the rows they updated into this rank's copies
        torch.cuda.synchronize()
        epr = cfg.num_experts // world
        for n in ("w13", "w2"):
            a, b = getattr(arms["1"], n).detach().float(), getattr(arms["0"], n).detach().float()
            moved = (b - before[n]).abs().max().item()
            assert moved > 1e-3, f"{n}: the update must be visible ({moved})"
            err = (a - b).abs().max().item()
            assert err < 0.05 * moved + 3e-4, f"rank {rank} {n}: pushed sum {err} away from the all-reduce arm (weights moved {moved})"
            copies = [torch.empty_like(a[epr:]) for _ in range(world)]
            dist.all_gather(copies, a[epr:].contiguous())
            assert all(torch.equal(c, copies[0]) for c in copies), f"{n}: the copies must stay identical on every rank"

    # ---- experts placed by expected load, then the layer rebalances itself from its own routing -----------------
    # (copy slots start empty; rebalance() picks the shadows and spreads their rows over the ranks' copies)
    if world > 1 and cfg.num_experts // world > 1:
        pl = MoELayer(cfg, heap, rank, world, device=dev, seed=4, fused_sgd_lr=0.0, name="moe_pl", placement="balanced",
                      shadow_experts=[-1, -1])
        bpl = BaselineMoELayer(cfg, rank, world, device=dev, seed=4, placement="balanced")
        F = cfg.ffn
        for step in range(3):
            g = torch.Generator(device=dev).manual_seed(130 + step * 10 + rank)
            x = torch.randn(cfg.tokens, cfg.hidden, generator=g, device=dev).to(torch.bfloat16)
            xa, xb = x.clone().requires_grad_(True), x.clone().requires_grad_(True)
            oa, ob = pl(xa), bpl(xb)
            (oa.float().pow(2).mean()).backward()
            (ob.float().pow(2).mean()).backward()
            torch.cuda.synchronize()
            heap.check_status("moe placement")

            def close(a, b, what, tol=5e-2):
                err = (a.float() - b.float()).abs().max().item()
                den = b.float().abs().max().item() + 1e-6
                assert err < tol * den, f"rank {rank} step {step} placement {what}: err {err} vs {den}"

            close(oa, ob, "out")
            close(xa.grad, xb.grad, "dx")
            dg, du = gemm.deinterleave_gate_up(pl.w13.grad)
            for le, e in enumerate(pl.local_experts):           # same homes in both arms: local index le holds expert e
                slot = pl.epr + pl.cfg.shadow.index(e) if e in pl.cfg.shadow else le
                close(dg[slot], bpl.w13.grad[le, :F], f"dWgate expert {e}")
                close(du[slot], bpl.w13.grad[le, F:], f"dWup expert {e}")
                close(pl.w2.grad[slot], bpl.w2.grad[le], f"dW2 expert {e}")
            for m in (pl, bpl):
                m.zero_grad(set_to_none=True)
            if step == 0:
                chosen = pl.rebalance(tolerance=0.0)            # tolerance 0: shadows are chosen whenever a rank is above the mean
                rows = pl.ws.counts_now().sum().to(torch.float64).reshape(1)
        # after the rebalance every rank computes about the mean number of rows
        rows = pl.ws.counts_now().sum().to(torch.float64).reshape(1)
        hi = rows.clone(); dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        if any(e >= 0 for e in pl.cfg.shadow):
            assert float(hi) <= 1.15 * cfg.tokens * cfg.topk, (rank, float(hi), pl.cfg.shadow)

    # ---- DLRM: fused embedding-bag + all-to-all vs EmbeddingBag + NCCL ------------------------------------
    dcfg = DLRMConfig(num_tables=10, rows=4000, dim=128, pooling=20, global_batch=64 * world, lr=0.05)
    a = DLRM(dcfg, heap, rank, world, device=dev, seed=9)
    b = BaselineDLRM(dcfg, rank, world, device=dev, seed=9)
    b.tables.copy_(a.tables)
    b.bottom.load_state_dict(a.bottom.state_dict())
    b.top.load_state_dict(a.top.state_dict())
    oa_, ob_ = torch.optim.SGD(a.dense_parameters(), lr=dcfg.lr), torch.optim.SGD(b.dense_parameters(), lr=dcfg.lr)
    for step in range(3):
        d, i, l = synthetic_batch(dcfg, rank, world, dev, seed=step)
        la, lb = a.train_step(d, i, l, oa_), b.train_step(d, i, l, ob_)
        assert abs(float(la) - float(lb)) < 1e-4, (rank, step, float(la), float(lb))
    torch.cuda.synchronize()
    heap.check_status("dlrm")
    torch.testing.assert_close(a.tables, b.tables, rtol=1e-4, atol=1e-6)

    dist.barrier()
    if rank == 0:
        print("MULTIGPU-OK world", world, flush=True)
    import threading
    wd = threading.Timer(60.0, lambda: os._exit(0))     # the checks are done: teardown may not hang the job
    wd.daemon = True
    wd.start()
    heap.close()
    dist.destroy_process_group()
    wd.cancel()


if __name__ == "__main__":
    main()
