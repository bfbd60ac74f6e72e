"""Shadow experts: the slot arithmetic, the replicated initialisation and the gradient rule, checked on the CPU with the
plain-PyTorch expert function standing in for the grouped GEMMs (the kernels see slots as experts and do not change)."""
import torch

from fuselink_b200.models.moe import MoELayer
from fuselink_b200.ops import gemm, ref
from fuselink_b200.ops.moe import MoEConfig, slot_table


def test_slot_table_sends_ordinary_rows_to_the_owner_and_shadowed_rows_nowhere():
    E, W, shadow = 8, 4, (5, 0)
    real, spr = E // W, E // W + len(shadow)
    for rank in range(W):
        t = slot_table(E, W, shadow, rank)
        assert t[0] == -1 and t[E + 1] == -1                       # ids out of range, after clamp(e, -1, E) + 1
        slots = t[1:E + 1].tolist()
        assert len(set(slots)) == E                                 # no two experts share a slot
        for e, s in enumerate(slots):
            dest, local = divmod(s, spr)
            if e in shadow:
                assert dest == rank and local == real + shadow.index(e)
            else:
                assert dest == e // real and local == e % real
    bad = torch.tensor([-7, 99, 3])
    assert slot_table(E, W, shadow, 0)[(bad.clamp(-1, E) + 1).long()].tolist()[:2] == [-1, -1]


def test_shadow_choice_follows_the_router_bias_and_copies_start_equal():
    cfg = MoEConfig(hidden=128, ffn=256, num_experts=8, topk=2, tokens=16)
    W = 4
    layers = [MoELayer(cfg, None, r, W, device="cpu", zipf_s=1.2, seed=5, shadow_experts=2) for r in range(W)]
    assert all(l.cfg.shadow == (0, 1) for l in layers)              # Zipf bias: experts 0 and 1 are the hot ones
    assert cfg.shadow == ()                                         # the caller's config is not modified
    assert layers[0].w13.shape[0] == 2 + 2 and layers[0].w2.shape[0] == 4
    for l in layers:                                                # every copy equals the owner's expert
        assert torch.equal(l.w13[2], layers[0].w13[0]) and torch.equal(l.w13[3], layers[0].w13[1])
        assert torch.equal(l.w2[2], layers[0].w2[0]) and torch.equal(l.w2[3], layers[0].w2[1])
    explicit = MoELayer(cfg, None, 1, W, device="cpu", zipf_s=None, seed=5, shadow_experts=[6])
    assert explicit.cfg.shadow == (6,) and torch.equal(explicit.w2[2], MoELayer(cfg, None, 3, W, device="cpu", seed=5).w2[0])
    plain = MoELayer(cfg, None, 1, W, device="cpu", seed=5)
    assert plain.cfg.shadow == () and plain.w13.shape[0] == 2 and torch.equal(plain.w13.data, layers[1].w13.data[:2])


def test_slot_level_computation_equals_the_unshadowed_one_and_gradients_add_up():
    """What the fused path does with slots, in plain PyTorch: every rank's rows for a shadowed expert run through that
    rank's copy.  Outputs equal the ordinary formulation; the gradient of the expert is the sum of the copies' gradients
    (which is why they are all-reduced), and the owner's own slot of a shadowed expert sees nothing."""
    torch.manual_seed(0)
    E, W, T, H, F, k = 8, 4, 24, 128, 256, 2
    cfg = MoEConfig(hidden=H, ffn=F, num_experts=E, topk=k, tokens=T)
    layers = [MoELayer(cfg, None, r, W, device="cpu", zipf_s=1.2, seed=9, shadow_experts=[0, 3]) for r in range(W)]
    real, spr = E // W, E // W + 2
    shadow = layers[0].cfg.shadow
    xs = [torch.randn(T, H) for _ in range(W)]
    routes = [layers[r].route(xs[r].to(torch.bfloat16)) for r in range(W)]
    # the experts, once each (fp32 leaves)
    wg_r, wu_r, w2_r = [], [], []
    for l in layers:
        g_, u_ = gemm.deinterleave_gate_up(l.w13.data[:real])
        wg_r.append(g_.float()); wu_r.append(u_.float()); w2_r.append(l.w2.data[:real].float())
    wg, wu, w2 = (torch.cat(v).clone().requires_grad_(True) for v in (wg_r, wu_r, w2_r))
    want = [ref.moe_forward(xs[r], routes[r][1], routes[r][0].detach().float(), wg, wu, w2) for r in range(W)]
    sum(o.sum() for o in want).backward()
    # all slots of all ranks (fp32 leaves): [W * spr, ...]
    sg_, su_, s2_ = [], [], []
    for l in layers:
        g_, u_ = gemm.deinterleave_gate_up(l.w13.data)
        sg_.append(g_.float()); su_.append(u_.float()); s2_.append(l.w2.data.float())
    sg, su, s2 = (torch.cat(v).clone().requires_grad_(True) for v in (sg_, su_, s2_))
    got = []
    for r in range(W):
        slots = slot_table(E, W, shadow, r)[(routes[r][1].clamp(-1, E) + 1).long()]
        got.append(ref.moe_forward(xs[r], slots, routes[r][0].detach().float(), sg, su, s2))
    sum(o.sum() for o in got).backward()
    for r in range(W):
        assert torch.allclose(got[r], want[r], atol=1e-5)
    grads = s2.grad.view(W, spr, H, F)
    for e in range(E):
        owner, local = divmod(e, real)
        if e in shadow:
            j = shadow.index(e)
            assert torch.allclose(grads[:, real + j].sum(0), w2.grad[e], atol=1e-5)      # sum over the copies
            assert grads[owner, local].abs().max() == 0                                   # the owner's own slot is idle
        else:
            assert torch.allclose(grads[owner, local], w2.grad[e], atol=1e-5)


def test_sync_shadow_to_real_refreshes_the_owners_slot():
    cfg = MoEConfig(hidden=128, ffn=256, num_experts=4, topk=2, tokens=8)
    l = MoELayer(cfg, None, 1, 2, device="cpu", seed=1, shadow_experts=[2, 0])     # rank 1 owns experts 2 and 3
    with torch.no_grad():
        l.w13[2].add_(1.0); l.w2[2].add_(1.0)                                       # its copy of expert 2 has been trained
        l.w13[3].add_(5.0)                                                          # copy of expert 0: not this rank's to export
    before = l.w13[1].clone()
    l.sync_shadow_to_real()
    assert torch.equal(l.w13[0], l.w13[2]) and torch.equal(l.w2[0], l.w2[2]) and torch.equal(l.w13[1], before)


def _reshadow_worker(rank, world, port, out_dir):
    import os
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    cfg = MoEConfig(hidden=128, ffn=256, num_experts=4, topk=2, tokens=8)
    l = MoELayer(cfg, None, rank, world, device="cpu", seed=3, shadow_experts=[0])        # expert 0 lives on rank 0
    with torch.no_grad():
        l.w2[2].add_(0.5)                       # every rank trained its copy of expert 0 (identically, as the all-reduce ensures)
        if rank == 1:
            l.w2[0].mul_(2.0)                   # rank 1 trained its own expert 2
    # this batch's routing: expert 2 (owned by rank 1) is now the busiest one over both ranks
    idx = torch.tensor([[2, 3], [2, 1]]) if rank == 0 else torch.tensor([[2, 0], [2, 3]])
    chosen = l.reshadow(idx)
    torch.save({"chosen": chosen, "w2": l.w2.data.clone(), "shadow": l.cfg.shadow}, os.path.join(out_dir, f"r{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


def test_reshadow_moves_the_weights_between_owners_and_copies(tmp_path):
    import os
    import socket
    import torch.multiprocessing as mp
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    mp.spawn(_reshadow_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    r0, r1 = (torch.load(os.path.join(str(tmp_path), f"r{r}.pt")) for r in range(2))
    assert r0["chosen"] == r1["chosen"] == (2,) and r0["shadow"] == (2,)
    cfg = MoEConfig(hidden=128, ffn=256, num_experts=4, topk=2, tokens=8)
    fresh = [MoELayer(cfg, None, r, 2, device="cpu", seed=3) for r in range(2)]
    # expert 0's owner took the trained copy back into the expert's own slot
    assert torch.allclose(r0["w2"][0].float(), fresh[0].w2.data[0].float() + 0.5, atol=1e-2)
    # both copy slots now hold expert 2 as its owner (rank 1) had it
    want = fresh[1].w2.data[0].float() * 2.0
    assert torch.allclose(r0["w2"][2].float(), want, atol=1e-2) and torch.equal(r0["w2"][2], r1["w2"][2])


def test_choice_of_shadows_stops_when_the_load_is_level_enough():
    from fuselink_b200.ops.moe import busiest_rank_load, choose_shadows
    load = torch.tensor([4300., 2000., 1100., 900., 700., 600., 500., 400.])       # 8 ranks, one expert each; mean 1312.5
    assert busiest_rank_load(load.tolist(), 8, ()) == 4300
    assert busiest_rank_load(load.tolist(), 8, (0,)) == 2000 + 4300 / 8
    assert choose_shadows(load, 3) == (0, 1, 2)                                    # no tolerance given: fill every slot
    assert choose_shadows(load, 4, world=8, tolerance=0.6) == (0, 1, -1, -1)       # 1100 + 6300 / 8 = 1887 < 1.6 x mean
    assert choose_shadows(load, 4, world=8, tolerance=0.05) == (0, 1, 2, 3)        # slots run out first
    assert choose_shadows(torch.full((8,), 100.), 4, world=8, tolerance=0.1) == (-1, -1, -1, -1)   # balanced router: no copies
    # two ranks, four experts each: rank 0 owns the hot ones
    assert choose_shadows(torch.tensor([500., 400., 300., 200., 50., 50., 50., 50.]), 3, world=2, tolerance=0.2) == (0, 1, -1)


def test_empty_copy_slots_in_the_table_and_the_layer():
    t = slot_table(8, 4, (5, -1), 2)
    assert t[6] == 2 * 4 + 2 and sorted(t[1:9].tolist()) == sorted([0, 1, 4, 5, 8, 9, 10, 12, 13][:0] + t[1:9].tolist())
    assert (t[1:9] == 2 * 4 + 3).sum() == 0                                        # nothing maps to the empty slot
    import pytest
    with pytest.raises(AssertionError):
        slot_table(8, 4, (-1, 5), 2)                                               # slots in use come first
    cfg = MoEConfig(hidden=128, ffn=256, num_experts=4, topk=2, tokens=8)
    l = MoELayer(cfg, None, 0, 1, device="cpu", seed=1, shadow_experts=[2, 3])
    l.set_shadows([-1, 3])                                                         # normalised: the slot in use first
    assert l.cfg.shadow == (3, -1) and torch.equal(l.w2[4], l.w2[3])
    l.reshadow(torch.tensor([[0, 1], [2, 3], [0, 2], [1, 3]]), tolerance=0.5)     # one rank: always level
    assert l.cfg.shadow == (-1, -1)


def test_spread_plan_levels_the_ranks_and_the_pattern_follows_it():
    """Zipf-skewed loads on 2, 4 and 8 ranks: with as few shadows as the tolerance asks for and their rows split by the plan
    every rank computes the mean within the tolerance; the per-token pattern realises the plan's shares."""
    import torch
    from fuselink_b200.ops import moe as M
    L = [45754, 28357, 18115, 12716, 9339, 6862, 5565, 4364]
    for W, want in ((2, 0), (4, 1), (8, 3)):
        pl = M.balanced_placement(L, W)
        load = [[x / W for x in L] for _ in range(W)]
        ch = M.choose_shadows(torch.tensor(L, dtype=torch.float64), 4, W, 0.05, pl, spread=True)
        assert sum(e >= 0 for e in ch) == want, (W, ch)
        plan = M.spread_plan(load, W, ch, pl)
        own = M.owned_rows(L, W, ch, pl)
        made = [sum(load[r][e] for e in ch if e >= 0) for r in range(W)]
        tot = [own[d] + sum(made[r] * plan[r][d] for r in range(W)) for d in range(W)]
        mean = sum(L) / W
        assert max(tot) <= 1.05 * mean + 1 and abs(sum(tot) - sum(L)) < 1e-6 * sum(L)
        for r in range(W):
            assert abs(sum(plan[r]) - 1.0) < 1e-9 and min(plan[r]) >= 0
            pat = M.spread_pattern(plan[r], 8192, r)
            for d in range(W):
                assert abs(float((pat == d - r).double().mean()) - plan[r][d]) < 2e-3
    # nothing shadowed, or nothing to move: rows stay where they are
    assert M.spread_plan([[1.0] * 8] * 2, 2, (), ()) == [[1.0, 0.0], [0.0, 1.0]]
