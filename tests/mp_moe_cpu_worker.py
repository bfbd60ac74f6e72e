"""Worker of tests/test_kernel_model_cpu.py::test_expert_parallel_step_between_processes: the expert-parallel MoE step with
shadow experts between REAL processes on a machine without a GPU.  The symmetric heap is memfd-backed host memory shared by
the ranks, the device entry points are the host model of tests/cpu_kernel_model.py (its barriers and waits are real), the
sum of the shadow experts' gradients is a real all-reduce (gloo) and a change of the shadowed experts a real broadcast.
The oracle is the whole layer in fp32 autograd, rebuilt on every rank from all-gathered inputs, routes and weights."""
import datetime
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import torch
import torch.distributed as dist


def gather(t):
    out = [torch.empty_like(t) for _ in range(dist.get_world_size())]
    dist.all_gather(out, t.contiguous())
    return out


def close(a, b, what, tol=4e-2):
    err = (a.float() - b.float()).abs().max().item()
    assert err < tol * (b.float().abs().max().item() + 1e-4), f"rank {dist.get_rank()} {what}: err {err} vs max {b.float().abs().max().item()}"


def main():                      # the change of shadows below names expert 5: shapes with at least 6 experts
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=120))
    import cpu_kernel_model
    from fuselink_b200.models.moe import MoELayer
    from fuselink_b200.ops import gemm, moe as M, ref
    from fuselink_b200.parallel.symm import SymmetricHeap
    E, T, k, H, F = int(os.environ.get("FL_MOE_E", "8")), int(os.environ.get("FL_MOE_T", "32")), int(os.environ.get("FL_MOE_K", "2")), 128, 256
    epr = E // world
    cfg = M.MoEConfig(hidden=H, ffn=F, num_experts=E, topk=k, tokens=T)
    with cpu_kernel_model.installed(single_process=False, lock_path=os.environ["FL_MODEL_LOCK"]) as model:
        model.wait_limit_s = 20.0
        heap = SymmetricHeap.create(48 << 20, device=-1)
        for sgd in (0.0, 0.05):
            layer = MoELayer(cfg, heap, rank, world, device="cpu", zipf_s=1.2, seed=11, fused_sgd_lr=sgd, name=f"l{sgd}", shadow_experts=2,
                             placement=os.environ.get("FL_MOE_PLACEMENT") or None)
            shadow = layer.cfg.shadow
            assert shadow == (0, 1)
            pushed = os.environ.get("FUSELINK_PUSH_REDUCE", "1") != "0" and (2 * F) % world == 0 and H % world == 0
            assert (layer.ws.push is not None) == pushed, "the copies' gradients are summed by the library's own kernels when they can be"
            # the experts themselves, once each, as fp32 leaves (every rank builds the same oracle)
            wg_, wu_ = gemm.deinterleave_gate_up(layer.w13.data[:epr])
            order = [layer.home(e)[0] * epr + layer.home(e)[1] for e in range(E)]      # gathered in slot order, wanted by expert id
            wg, wu, w2 = (torch.cat(gather(t.float()))[order].clone().requires_grad_(True) for t in (wg_, wu_, layer.w2.data[:epr]))
            for step in range(2):
                g = torch.Generator().manual_seed(100 * step + rank)
                x = torch.randn(T, H, generator=g).to(torch.bfloat16)
                dout = torch.randn(T, H, generator=g).to(torch.bfloat16)
                xa = x.clone().requires_grad_(True)
                with torch.no_grad():
                    w_, idx = layer.route(x)
                wa = w_.clone().requires_grad_(True)
                out = M.MoEFunction.apply(xa, wa, idx, layer.w13, layer.w2, layer.ws, sgd)
                (out.float() * dout.float()).sum().backward()
                heap.check_status(f"step {step}")
                # ---- oracle over all ranks' tokens
                xs, douts, ws_, idxs = gather(x), gather(dout), gather(w_), gather(idx)
                xr = [t.float().requires_grad_(True) for t in xs]
                wr = [t.float().requires_grad_(True) for t in ws_]
                for t in (wg, wu, w2):
                    t.grad = None
                refs = [ref.moe_forward(xr[r], idxs[r], wr[r], wg, wu, w2) for r in range(world)]
                sum((refs[r] * douts[r].float()).sum() for r in range(world)).backward()
                close(out, refs[rank], "out", 3e-2)
                close(xa.grad, xr[rank].grad, "dx")
                close(wa.grad, wr[rank].grad, "dw")
                slot_of = lambda e: epr + shadow.index(e) if e in shadow else layer.home(e)[1]
                mine = [e for e in range(E) if e in shadow or layer.home(e)[0] == rank]
                if not sgd:
                    dg, du = gemm.deinterleave_gate_up(layer.w13.grad)
                    for e in mine:
                        close(dg[slot_of(e)], wg.grad[e], f"dWgate expert {e}")
                        close(du[slot_of(e)], wu.grad[e], f"dWup expert {e}")
                        close(layer.w2.grad[slot_of(e)], w2.grad[e], f"dW2 expert {e}")
                    layer.zero_grad(set_to_none=True)
                else:
                    layer.weights_ready()       # pushed sums: the rows of this rank's copies are written by the ranks that summed them
                    with torch.no_grad():
                        for t in (wg, wu, w2):
                            t -= sgd * t.grad
                    g_, u_ = gemm.deinterleave_gate_up(layer.w13.data)
                    for e in mine:
                        close(g_[slot_of(e)], wg.detach()[e], f"Wgate expert {e} after the update", 2e-2)
                        close(layer.w2.data[slot_of(e)], w2.detach()[e], f"W2 expert {e} after the update", 2e-2)
                    copies = gather(layer.w2.data[epr:].float())
                    assert all(torch.equal(c, copies[0]) for c in copies), "the copies must stay identical on every rank"
            if sgd:
                # choose the shadows again from the last routing (same Zipf bias: same experts), then force another pair
                assert layer.reshadow()[:2] == (0, 1)                # no tolerance given: both copy slots are filled, hottest first
                layer.set_shadows((5, 0))
                assert layer.ws.cfg.shadow == (5, 0) and layer.cfg.shadow == (5, 0)
                owner5 = gather(layer.w2.data[layer.home(5)[1]].float())[layer.home(5)[0]]
                assert torch.equal(layer.w2.data[epr].float(), owner5), "expert 5 must have travelled from its owner into the copy slot"
                if rank == layer.home(1)[0]:                         # expert 1 is no longer shadowed: its owner took the trained copy back
                    close(layer.w2.data[layer.home(1)[1]], w2.detach()[1], "W2 of the expert that went home", 2e-2)
                x = torch.randn(T, H).to(torch.bfloat16)
                with torch.no_grad():
                    w_, idx = layer.route(x)
                    out = M.MoEFunction.apply(x, w_, idx, layer.w13, layer.w2, layer.ws, 0.0)
                heap.check_status("after the change")
                assert int(layer.ws.counts_now()[epr]) == int((idx == 5).sum()) and int(layer.ws.counts_now()[epr + 1]) == int((idx == 0).sum())
                # the layer evens out the ranks by itself: shadows from the observed routing, their rows spread over the copies
                chosen = layer.rebalance(tolerance=0.0)
                assert layer.cfg.shadow == chosen == layer.ws.cfg.shadow
                wg_, wu_ = gemm.deinterleave_gate_up(layer.w13.data[:epr])      # the owners hold the current weights again
                wg, wu, w2 = (torch.cat(gather(t.float()))[order].clone().requires_grad_(True) for t in (wg_, wu_, layer.w2.data[:epr]))
                g = torch.Generator().manual_seed(4242 + rank)
                x = torch.randn(T, H, generator=g).to(torch.bfloat16)
                dout = torch.randn(T, H, generator=g).to(torch.bfloat16)
                xa = x.clone().requires_grad_(True)
                with torch.no_grad():
                    w_, idx = layer.route(x)
                wa = w_.clone().requires_grad_(True)
                layer.zero_grad(set_to_none=True)
                out = M.MoEFunction.apply(xa, wa, idx, layer.w13, layer.w2, layer.ws, 0.0)
                (out.float() * dout.float()).sum().backward()
                heap.check_status("after the rebalance")
                xs, douts, ws_, idxs = gather(x), gather(dout), gather(w_), gather(idx)
                xr = [t.float().requires_grad_(True) for t in xs]
                wr = [t.float().requires_grad_(True) for t in ws_]
                refs = [ref.moe_forward(xr[r], idxs[r], wr[r], wg, wu, w2) for r in range(world)]
                sum((refs[r] * douts[r].float()).sum() for r in range(world)).backward()
                close(out, refs[rank], "out after the rebalance", 3e-2)
                close(xa.grad, xr[rank].grad, "dx after the rebalance")
                close(wa.grad, wr[rank].grad, "dw after the rebalance")
                dg, du = gemm.deinterleave_gate_up(layer.w13.grad)
                for e in range(E):
                    if e in chosen or layer.home(e)[0] == rank:
                        sl = epr + chosen.index(e) if e in chosen else layer.home(e)[1]
                        close(dg[sl], wg.grad[e], f"dWgate expert {e} after the rebalance")
                        close(layer.w2.grad[sl], w2.grad[e], f"dW2 expert {e} after the rebalance")
                rows = gather(layer.ws.counts_now().sum().reshape(1).to(torch.int64))
                assert sum(int(r) for r in rows) == world * T * k
        dist.barrier()
        print(f"MOE-MP-OK rank {rank}", flush=True)
        heap.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
