"""MoE expert-parallel forward/backward on one GPU with 1, 2 and 4 virtual ranks, against the fp32 oracle."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _run(world, T=256, H=256, Fd=512, E=8, k=2, sgd=0.0, steps=1, fp8=False, shadow=(), device="cuda", placement=None, spread=None):
    from fuselink_b200.models.moe import MoELayer
    from fuselink_b200.ops import gemm, moe as M, ref
    from fuselink_b200.parallel.symm import SymmetricHeap
    cfg = M.MoEConfig(hidden=H, ffn=Fd, num_experts=E, topk=k, tokens=T, fp8=fp8)
    ftol = 4.0 if fp8 else 1.0      # e4m3 operands: a few percent of relative error per GEMM
    heaps = SymmetricHeap.emulated(world, 64 << 20)
    sync = torch.cuda.synchronize if device == "cuda" else (lambda: None)
    try:
        layers = [MoELayer(cfg, heaps[r], r, world, device=device, seed=3, fused_sgd_lr=sgd, name="m", shadow_experts=list(shadow), placement=placement)
                  for r in range(world)]
        epr = E // world
        for r in range(1, world):
            layers[r].router.data.copy_(layers[0].router.data)
        if spread is not None:          # share[r][d]: fraction of rank r's shadow rows that rank d's copy computes
            for r in range(world):
                layers[r].ws.set_spread(M.spread_pattern(spread[r], T, r))
        wg_all, wu_all, w2_all = [], [], []
        for l in layers:
            g_, u_ = gemm.deinterleave_gate_up(l.w13.data[:epr])          # the experts themselves; copies of shadowed ones follow
            wg_all.append(g_.float()); wu_all.append(u_.float()); w2_all.append(l.w2.data[:epr].float())
        wg, wu, w2 = (torch.cat(v) for v in (wg_all, wu_all, w2_all))     # in slot order: rank 0's experts, rank 1's, ...
        if placement is not None:                                         # the oracle wants them by expert id
            order = [layers[0].home(e)[0] * epr + layers[0].home(e)[1] for e in range(E)]
            wg, wu, w2 = wg[order], wu[order], w2[order]
        wg, wu, w2 = (t.clone().requires_grad_(True) for t in (wg, wu, w2))
        for step in range(steps):
            gen = torch.Generator(device=device).manual_seed(100 + step)
            xs = [torch.randn(T, H, generator=gen, device=device).to(torch.bfloat16) for _ in range(world)]
            douts = [torch.randn(T, H, generator=gen, device=device).to(torch.bfloat16) for _ in range(world)]
            with torch.no_grad():
                routes = [layers[r].route(xs[r]) for r in range(world)]
            wss = [l.ws for l in layers]
            # forward, phase by phase over the virtual ranks
            for r in range(world):
                M.moe_forward_dispatch(wss[r], xs[r], routes[r][1].contiguous())
            for r in range(world):
                M.moe_forward_experts(wss[r], layers[r].w13.data, layers[r].w2.data)
            outs = [M.moe_forward_combine(wss[r], routes[r][0].contiguous()) for r in range(world)]
            sync()
            for h in heaps:
                h.check_status("forward")
            total = sum(int(w_.counts_now().sum()) for w_ in wss)
            assert total == world * T * k
            # oracle (fp32, autograd)
            xr = [x.float().requires_grad_(True) for x in xs]
            wr = [routes[r][0].detach().clone().requires_grad_(True) for r in range(world)]
            for t in (wg, wu, w2):
                t.grad = None
            refs = [ref.moe_forward(xr[r], routes[r][1], wr[r], wg, wu, w2) for r in range(world)]
            for r in range(world):
                err = (outs[r].float() - refs[r]).abs().max().item()
                assert err < ftol * 3e-2 * (refs[r].abs().max().item() + 1e-3), f"forward rank {r}: {err}"
            sum((refs[r] * douts[r].float()).sum() for r in range(world)).backward()
            # backward
            dws = [M.moe_backward_dispatch(wss[r], douts[r], routes[r][1].contiguous(), routes[r][0].contiguous()) for r in range(world)]
            grads = [M.moe_backward_experts(wss[r], layers[r].w13.data, layers[r].w2.data, sgd, True) for r in range(world)]
            if any(e >= 0 for e in shadow) and not isinstance(wss[0].pending_shadow[0], int):
                # (an int: the GEMMs have pushed the copies' gradient rows to the ranks that sum them -- fused update)
                # the ranks are emulated on one GPU: the sum over ranks that NCCL would do is done here
                totals = [sum(wss[r].pending_shadow[0][i] for r in range(world)) for i in range(2)]
                for w_ in wss:
                    w_.reduce_shadow_grads = lambda ws_, gs, totals=totals: [g.copy_(t) for g, t in zip(gs, totals)]
            dxs = [M.moe_backward_finish(wss[r], True) for r in range(world)]
            for r in range(world):
                M.moe_backward_complete(wss[r])
            sync()
            for h in heaps:
                h.check_status("backward")

            def close(a, b, what, tol=4e-2):
                err = (a.float() - b).abs().max().item()
                assert err < ftol * tol * (b.abs().max().item() + 1e-4), f"{what}: err {err} ref max {b.abs().max().item()}"

            for r in range(world):
                close(dxs[r], xr[r].grad, f"dx rank {r}")
                close(dws[r], wr[r].grad, f"dw rank {r}")
            # slot -> expert: a rank's own experts, then its copies of the shadowed ones (whose own slots stay idle)
            own = lambda r: layers[r].local_experts                  # in slot order; r * epr ... in the default placement
            pick = lambda r: [i for i, e in enumerate(own(r)) if e not in shadow]
            plain = not shadow and placement is None
            if plain and not sgd:
                for r in range(world):
                    dg, du = gemm.deinterleave_gate_up(grads[r][0])
                    close(dg, wg.grad[r * epr:(r + 1) * epr], f"dWgate rank {r}")
                    close(du, wu.grad[r * epr:(r + 1) * epr], f"dWup rank {r}")
                    close(grads[r][1], w2.grad[r * epr:(r + 1) * epr], f"dW2 rank {r}")
            elif plain:
                with torch.no_grad():
                    for t in (wg, wu, w2):
                        t -= sgd * t.grad
                for r in range(world):
                    g_, u_ = gemm.deinterleave_gate_up(layers[r].w13.data)
                    close(g_, wg.detach()[r * epr:(r + 1) * epr], f"Wgate after sgd rank {r}", 2e-2)
                    close(layers[r].w2.data, w2.detach()[r * epr:(r + 1) * epr], f"W2 after sgd rank {r}", 2e-2)
            elif not sgd:
                for r in range(world):
                    dg, du = gemm.deinterleave_gate_up(grads[r][0])
                    for i in pick(r):
                        close(dg[i], wg.grad[own(r)[i]], f"dWgate rank {r} slot {i}")
                        close(du[i], wu.grad[own(r)[i]], f"dWup rank {r} slot {i}")
                        close(grads[r][1][i], w2.grad[own(r)[i]], f"dW2 rank {r} slot {i}")
                    for j, e in enumerate(shadow):                      # summed over the ranks: the expert's whole gradient
                        if e < 0:                                       # an empty copy slot
                            assert grads[r][1][epr + j].abs().max() == 0 and dg[epr + j].abs().max() == 0
                            continue
                        close(dg[epr + j], wg.grad[e], f"dWgate shadow {e} on rank {r}")
                        close(du[epr + j], wu.grad[e], f"dWup shadow {e} on rank {r}")
                        close(grads[r][1][epr + j], w2.grad[e], f"dW2 shadow {e} on rank {r}")
            else:
                with torch.no_grad():
                    for t in (wg, wu, w2):
                        t -= sgd * t.grad
                for r in range(world):
                    g_, u_ = gemm.deinterleave_gate_up(layers[r].w13.data)
                    for i in pick(r):
                        close(g_[i], wg.detach()[own(r)[i]], f"Wgate after sgd rank {r} slot {i}", 2e-2)
                        close(layers[r].w2.data[i], w2.detach()[own(r)[i]], f"W2 after sgd rank {r} slot {i}", 2e-2)
                    for j, e in enumerate(shadow):
                        if e < 0:
                            continue
                        close(g_[epr + j], wg.detach()[e], f"Wgate copy of {e} after sgd rank {r}", 2e-2)
                        close(layers[r].w2.data[epr + j], w2.detach()[e], f"W2 copy of {e} after sgd rank {r}", 2e-2)
                        assert torch.equal(layers[r].w2.data[epr + j], layers[0].w2.data[epr + j]), "copies must stay identical"
    finally:
        for h in heaps:
            h.close()


@pytest.mark.parametrize("world", [1, 2, 4])
def test_moe_fwd_bwd(world):
    _run(world)


@pytest.mark.parametrize("world", [1, 2])
def test_moe_fwd_bwd_fp8_block_scaled(world):
    _run(world, fp8=True)


@pytest.mark.parametrize("world,shadow", [(2, (0,)), (4, (0, 5)), (1, (2,)), (2, (4, -1))])
def test_moe_shadow_experts(world, shadow):
    """Hot experts replicated on every rank: same outputs and gradients as without, the copies' gradients summed."""
    _run(world, shadow=shadow)


@pytest.mark.parametrize("world,placement", [(2, "balanced"), (4, "balanced"), (2, (7, 6, 5, 4, 3, 2, 1, 0))])
def test_moe_expert_placement(world, placement):
    """Experts owned out of order: one index gather in front of the dispatch kernel, everything else as in test_moe_fwd_bwd."""
    _run(world, placement=placement)
    _run(world, placement=placement, sgd=0.05, steps=2)


def test_moe_shadow_experts_two_steps_fused_sgd():
    _run(2, sgd=0.05, steps=2, shadow=(1,))


@pytest.mark.parametrize("world,shadow,spread", [
    (2, (0,), [[0.5, 0.5], [0.25, 0.75]]),
    (4, (0, 5), [[1, 0, 0, 0], [0.2, 0.3, 0.5, 0], [0, 0, 0.4, 0.6], [0.25, 0.25, 0.25, 0.25]]),
    (2, (4, -1), [[0.0, 1.0], [1.0, 0.0]]),
])
def test_moe_shadow_rows_spread_over_the_copies(world, shadow, spread):
    """A shadowed expert's rows may be computed by any rank's copy: same outputs and gradients whatever the split."""
    _run(world, shadow=shadow, spread=spread)
    _run(world, shadow=shadow, spread=spread, sgd=0.05, steps=2)


def test_moe_two_steps_fused_sgd():
    _run(2, sgd=0.05, steps=2)


def test_moe_layer_autograd_single_rank():
    from fuselink_b200.models.moe import smoke_step
    loss = smoke_step("cuda:0")
    assert loss == loss
