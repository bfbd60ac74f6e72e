"""Host-side logic of the model layers as gloo ranks on the CPU: the expert-parallel MoE layer and the
table-wise sharded DLRM give the same result at world 1 and world 2; checkpoint round trip."""
import os
import socket
import tempfile

import pytest

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _moe_worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from fuselink_b200.models.moe import MoELayer
    from fuselink_b200.ops.moe import MoEConfig
    cfg = MoEConfig(hidden=64, ffn=128, num_experts=4, topk=2, tokens=24)
    layer = MoELayer(cfg, None, rank, world, device="cpu", seed=5)
    g = torch.Generator().manual_seed(100 + rank)
    x = torch.randn(cfg.tokens, cfg.hidden, generator=g).to(torch.bfloat16)
    out = layer(x)
    torch.save({"x": x, "out": out, "w13": layer.w13.data, "w2": layer.w2.data, "router": layer.router.data}, os.path.join(out_dir, f"r{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


def test_moe_layer_world2_matches_world1_on_cpu():
    from fuselink_b200.models.moe import MoELayer
    from fuselink_b200.ops import gemm, ref
    from fuselink_b200.ops.moe import MoEConfig
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_moe_worker, args=(2, _free_port(), d), nprocs=2, join=True)
        parts = [torch.load(os.path.join(d, f"r{r}.pt")) for r in range(2)]
    cfg = MoEConfig(hidden=64, ffn=128, num_experts=4, topk=2, tokens=24)
    w13 = torch.cat([p["w13"] for p in parts])
    w2 = torch.cat([p["w2"] for p in parts])
    wg, wu = gemm.deinterleave_gate_up(w13)
    single = MoELayer(cfg, None, 0, 1, device="cpu", seed=5)
    assert torch.equal(single.w13.data, w13), "expert init must not depend on the number of ranks"
    for r in range(2):
        x = parts[r]["x"]
        w, idx = single.route(x)
        want = ref.moe_forward(x, idx, w, wg, wu, w2)
        assert (parts[r]["out"].float() - want).abs().max() < 2e-2 * (want.abs().max() + 1e-3)


def _dlrm_worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from fuselink_b200.models.dlrm import DLRM, DLRMConfig, synthetic_batch
    cfg = DLRMConfig(num_tables=5, rows=300, dim=128, pooling=4, global_batch=32, lr=0.1)
    m = DLRM(cfg, None, rank, world, device="cpu", seed=3)
    opt = torch.optim.SGD(m.dense_parameters(), lr=cfg.lr)
    losses = []
    for step in range(3):
        d, i, l = synthetic_batch(cfg, rank, world, "cpu", seed=step)
        losses.append(float(m.train_step(d, i, l, opt)))
    torch.save({"tables": m.tables, "first": m.t_first, "losses": losses, "top0": m.top[0].weight.data}, os.path.join(out_dir, f"r{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


def test_dlrm_sharded_tables_update_consistently_on_cpu():
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_dlrm_worker, args=(2, _free_port(), d), nprocs=2, join=True)
        parts = [torch.load(os.path.join(d, f"r{r}.pt")) for r in range(2)]
    assert parts[0]["tables"].shape[0] == 3 and parts[1]["tables"].shape[0] == 2 and parts[1]["first"] == 3
    assert torch.allclose(parts[0]["top0"], parts[1]["top0"]), "dense replicas must stay in sync (all-reduced grads)"
    assert all(abs(l - 0.69) < 0.2 for l in parts[0]["losses"])


def test_table_split_and_zipf():
    from fuselink_b200.models.dlrm import table_split, zipf_indices
    assert [n for _, n in table_split(26, 8)] == [4, 4, 3, 3, 3, 3, 3, 3]
    idx = zipf_indices((20000,), 1000, 1.05, torch.Generator().manual_seed(0), "cpu")
    assert idx.min() >= 0 and idx.max() < 1000
    counts = torch.bincount(idx, minlength=1000).float()
    assert counts[0] > 5 * counts[50] > 0            # heavy head


def test_checkpoint_roundtrip_moe_state():
    from fuselink_b200.models.moe import MoELayer
    from fuselink_b200.ops.moe import MoEConfig
    cfg = MoEConfig(hidden=64, ffn=128, num_experts=4, topk=2, tokens=8)
    a = MoELayer(cfg, None, 0, 1, device="cpu", seed=1)
    b = MoELayer(cfg, None, 0, 1, device="cpu", seed=2)
    with tempfile.TemporaryDirectory() as d:
        torch.save(a.state_dict(), os.path.join(d, "ck.pt"))
        b.load_state_dict(torch.load(os.path.join(d, "ck.pt")))
    x = torch.randn(8, 64).to(torch.bfloat16)
    assert torch.equal(a(x), b(x))


def test_checkpoint_roundtrip_dlrm_includes_tables():
    from fuselink_b200.models.dlrm import DLRM, DLRMConfig, synthetic_batch
    cfg = DLRMConfig(num_tables=3, rows=200, dim=128, pooling=4, global_batch=16, lr=0.1)
    a, b = DLRM(cfg, None, 0, 1, device="cpu", seed=1), DLRM(cfg, None, 0, 1, device="cpu", seed=2)
    opt = torch.optim.SGD(a.dense_parameters(), lr=cfg.lr)
    a.train_step(*synthetic_batch(cfg, 0, 1, "cpu", seed=0), opt)          # tables now differ from their init
    with tempfile.TemporaryDirectory() as d:
        torch.save(a.state_dict(), os.path.join(d, "ck.pt"))
        b.load_state_dict(torch.load(os.path.join(d, "ck.pt")))
    assert "tables" in a.state_dict() and torch.equal(a.tables, b.tables)
    dense, idx, _ = synthetic_batch(cfg, 0, 1, "cpu", seed=3)
    assert torch.equal(a.dense_forward(dense, a._pooled_reference(idx)), b.dense_forward(dense, b._pooled_reference(idx)))


def test_gating_capacity_mask_matches_a_sequential_admission():
    from fuselink_b200.models.moe import capacity_keep_mask, expert_capacity
    g = torch.Generator().manual_seed(0)
    T, E, k = 200, 8, 2
    idx = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)])
    idx[:120, 0] = 3                                    # a hot expert
    cap = expert_capacity(T, E, k, 1.0)
    assert cap == 50
    keep = capacity_keep_mask(idx, E, cap)
    taken, want = [0] * E, torch.zeros(T, k, dtype=torch.bool)
    for j in range(k):                                  # all first choices, then all second choices, in token order
        for t in range(T):
            e = int(idx[t, j])
            want[t, j] = taken[e] < cap
            taken[e] += 1
    assert torch.equal(keep, want)
    assert keep[:50, 0].all() and not keep[50:120, 0].any()


def test_moe_layer_gating_options_on_cpu():
    from fuselink_b200.models.moe import MoELayer
    from fuselink_b200.ops.moe import MoEConfig
    cfg = MoEConfig(hidden=64, ffn=128, num_experts=4, topk=2, tokens=64)
    x = torch.randn(cfg.tokens, cfg.hidden, generator=torch.Generator().manual_seed(1)).to(torch.bfloat16)
    plain = MoELayer(cfg, None, 0, 1, device="cpu", seed=5, zipf_s=None)
    out0 = plain(x)
    assert 0.9 < float(plain.l_aux.detach()) < 4.0               # 1 when balanced, E when everything goes to one expert
    skew = MoELayer(cfg, None, 0, 1, device="cpu", seed=5, zipf_s=3.0)
    skew(x)
    assert float(skew.l_aux.detach()) > float(plain.l_aux.detach())
    # aux loss reaches the router
    (plain.l_aux * 0.01).backward()
    assert plain.router.grad is not None and plain.router.grad.abs().sum() > 0
    # dropping: choices over capacity contribute nothing
    drop = MoELayer(cfg, None, 0, 1, device="cpu", seed=5, zipf_s=3.0, capacity_factor=0.5, drop_tokens=True)
    out1 = drop(x)
    assert 0.0 < float(drop.dropped_fraction) < 1.0
    w, idx = drop.route(x)
    assert (w == 0).any() and torch.isfinite(out1.float()).all()
    # jitter only in training
    noisy = MoELayer(cfg, None, 0, 1, device="cpu", seed=5, zipf_s=None, noisy_gate="jitter", jitter_eps=0.5)
    noisy.eval()
    assert torch.equal(noisy(x), out0)
    noisy.train()
    w_a, _ = noisy.route(x)
    w_b, _ = noisy.route(x)
    assert not torch.equal(w_a, w_b)
    rs = MoELayer(cfg, None, 0, 1, device="cpu", seed=5, zipf_s=None, noisy_gate="rsample")
    _, i_a = rs.route(x)
    _, i_b = rs.route(x)
    assert not torch.equal(i_a, i_b)


def _moe_model_worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from fuselink_b200.models.moe_transformer import MOE_ZOO, MoETransformer
    B, S = 2, 16
    net = MoETransformer(MOE_ZOO["tiny_moe"], B * S, None, rank, world, device="cpu", seed=2)
    g = torch.Generator().manual_seed(40 + rank)
    tokens = torch.randint(0, 512, (B, S), generator=g)
    with torch.no_grad():
        logits = net(tokens)
    torch.save({"tokens": tokens, "logits": logits}, os.path.join(out_dir, f"r{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


def test_moe_transformer_trains_and_is_independent_of_the_expert_layout():
    from fuselink_b200.models.moe_transformer import MOE_ZOO, MoETransformer
    cfg = MOE_ZOO["tiny_moe"]
    B, S = 2, 16
    net = MoETransformer(cfg, B * S, None, 0, 1, device="cpu", seed=2)
    assert len(net.expert_parameters()) == 2 * cfg.layers
    assert {id(p) for p in net.expert_parameters()}.isdisjoint({id(p) for p in net.dense_parameters()})
    # a few SGD steps on one batch: the loss goes down and every kind of parameter receives a gradient
    g = torch.Generator().manual_seed(1)
    tokens = torch.randint(0, cfg.vocab, (B, S), generator=g)
    labels = torch.roll(tokens, -1, 1)
    opt = torch.optim.SGD(net.parameters(), lr=0.5)
    first = net.loss(tokens, labels)
    first.backward()
    for name in ("embed", "lm_head"):
        assert getattr(net, name).grad is not None
    blk = net.blocks[0]
    for p in (blk.wqkv, blk.wo, blk.moe.router, blk.moe.w13, blk.moe.w2):
        assert p.grad is not None and torch.isfinite(p.grad.float()).all() and p.grad.float().abs().sum() > 0
    opt.zero_grad()
    losses = [float(net.train_step(tokens, labels, opt)) for _ in range(12)]
    assert losses[-1] < losses[0] - 0.05, losses
    # expert parallelism does not change the function: two ranks with half of the experts each give the logits that one
    # rank with all experts gives on the same tokens
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_moe_model_worker, args=(2, _free_port(), d), nprocs=2, join=True)
        parts = [torch.load(os.path.join(d, f"r{r}.pt")) for r in range(2)]
    single = MoETransformer(cfg, B * S, None, 0, 1, device="cpu", seed=2)
    for p_ in parts:
        with torch.no_grad():
            want = single(p_["tokens"])
        assert (p_["logits"] - want).abs().max() < 5e-2 * max(1.0, want.abs().max().item())


def test_moe_training_script_runs_on_cpu_ranks():
    """experiments/run_moe_training.py on two gloo ranks: experts split over the ranks, dense gradients averaged."""
    import json
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(_free_port()), os.path.join(root, "experiments", "run_moe_training.py"), "--model", "tiny_moe",
           "--device", "cpu", "--steps", "4", "--log-every", "2", "--batch", "2", "--seq", "16"]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr[-3000:]
    lines = [json.loads(l) for l in out.stdout.splitlines() if l.startswith("{")]
    assert [l["step"] for l in lines] == [2, 4] and all(l["n_gpus"] == 2 and l["tokens_per_s"] > 0 and l["loss"] > 0 for l in lines)


def test_moe_training_checkpoint_resume_reproduces_the_run(tmp_path):
    """4 steps in one go == 2 steps, checkpoint, resume, 2 more steps (same seed, same data order is not required: the
    check is that the resumed model continues from the saved weights, so its first logged loss differs from a fresh run's)."""
    import json
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = os.path.join(root, "experiments", "run_moe_training.py")
    base = [sys.executable, script, "--model", "tiny_moe", "--device", "cpu", "--batch", "2", "--seq", "16", "--lr", "0.5", "--log-every", "1"]
    ck = str(tmp_path / "ck")
    a = subprocess.run(base + ["--steps", "3", "--checkpoint", ck], capture_output=True, text=True, timeout=300)
    assert a.returncode == 0 and os.path.exists(ck + ".rank0"), a.stderr[-2000:]
    fresh = subprocess.run(base + ["--steps", "1"], capture_output=True, text=True, timeout=300)
    resumed = subprocess.run(base + ["--steps", "1", "--resume", ck], capture_output=True, text=True, timeout=300)
    first = lambda r: json.loads([l for l in r.stdout.splitlines() if l.startswith("{")][0])["loss"]
    run3 = [json.loads(l)["loss"] for l in a.stdout.splitlines() if l.startswith("{")]
    assert first(fresh) == run3[0]                       # same seed, same first batch, same initial weights
    assert first(resumed) != first(fresh)                # the resumed run starts from the trained weights


def test_dlrm_training_script_two_ranks_checkpoint_and_resume(tmp_path):
    """experiments/run_dlrm_training.py on two gloo ranks: per-rank checkpoints (the tables differ), and a resumed run is
    the same as the run that was never interrupted."""
    import json
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = os.path.join(root, "experiments", "run_dlrm_training.py")
    port = _free_port()
    base = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1", "--master-port", str(port),
            script, "--device", "cpu", "--tables", "5", "--rows", "300", "--global-batch", "64", "--pooling", "4", "--lr", "0.5", "--log-every", "1"]
    ck = str(tmp_path / "ck")
    losses = lambda r: [json.loads(l)["loss"] for l in r.stdout.splitlines() if l.startswith("{")]
    whole = subprocess.run(base + ["--steps", "4"], capture_output=True, text=True, timeout=300)
    assert whole.returncode == 0, whole.stderr[-3000:]
    first = subprocess.run(base + ["--steps", "2", "--checkpoint", ck], capture_output=True, text=True, timeout=300)
    assert first.returncode == 0 and os.path.exists(ck + ".rank0") and os.path.exists(ck + ".rank1"), first.stderr[-3000:]
    rest = subprocess.run(base + ["--steps", "2", "--resume", ck], capture_output=True, text=True, timeout=300)
    assert rest.returncode == 0, rest.stderr[-3000:]
    assert [json.loads(l)["step"] for l in rest.stdout.splitlines() if l.startswith("{")] == [3, 4]
    assert losses(first) + losses(rest) == pytest.approx(losses(whole), abs=1e-5)
    wrong = subprocess.run([sys.executable, script, "--device", "cpu", "--tables", "5", "--rows", "300", "--global-batch", "64", "--pooling", "4",
                            "--steps", "1", "--resume", ck], capture_output=True, text=True, timeout=300)
    assert wrong.returncode != 0 and "written by 2 ranks" in wrong.stderr


def test_baseline_layer_gives_the_same_result_under_any_expert_placement():
    from fuselink_b200.models.moe_baseline import BaselineMoELayer
    from fuselink_b200.ops.moe import MoEConfig
    cfg = MoEConfig(hidden=128, ffn=256, num_experts=8, topk=2, tokens=64)
    a = BaselineMoELayer(cfg, 0, 1, device="cpu", seed=3)
    b = BaselineMoELayer(cfg, 0, 1, device="cpu", seed=3, placement=(7, 6, 5, 4, 3, 2, 1, 0))
    x = torch.randn(64, 128).to(torch.bfloat16)
    assert torch.equal(a(x), b(x)) and torch.equal(a.w2[0], b.w2[7]) and a.homes is None
    assert BaselineMoELayer(cfg, 0, 1, device="cpu", seed=3, placement="balanced").homes is None      # one rank: nothing to even out
