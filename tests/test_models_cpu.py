"""Host-side logic of the model layers as gloo ranks on the CPU: the expert-parallel MoE layer and the
table-wise sharded DLRM give the same result at world 1 and world 2; checkpoint round trip."""
import os
import socket
import tempfile

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
