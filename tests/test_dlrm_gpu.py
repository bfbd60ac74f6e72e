"""Fused embedding-bag + all-to-all kernels and the DLRM step on one GPU with virtual ranks."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _cfg(**kw):
    from fuselink_b200.models.dlrm import DLRMConfig
    base = dict(num_tables=7, rows=5000, dim=128, pooling=20, global_batch=512, lr=0.05)
    base.update(kw)
    return DLRMConfig(**base)


@pytest.mark.parametrize("world", [1, 2, 4])
def test_embbag_fwd_bwd_against_reference(world):
    from fuselink_b200.models.dlrm import DLRM, synthetic_batch
    from fuselink_b200.ops import ref
    from fuselink_b200.parallel.symm import SymmetricHeap
    cfg = _cfg()
    heaps = SymmetricHeap.emulated(world, 32 << 20)
    try:
        models = [DLRM(cfg, heaps[r], r, world, device="cuda", seed=1) for r in range(world)]
        batches = [synthetic_batch(cfg, r, world, "cuda", seed=5) for r in range(world)]
        full_tables = torch.cat([m.tables for m in models]).clone()
        full_idx = torch.cat([b[1] for b in batches])
        want = ref.embedding_bag_sum(full_tables, full_idx)                 # [B_global, T, D]
        for r in range(world):
            models[r].sparse_forward_launch(batches[r][1])
        pooled = [models[r].sparse_forward_wait() for r in range(world)]
        torch.cuda.synchronize()
        bl = cfg.global_batch // world
        for r in range(world):
            heaps[r].check_status()
            torch.testing.assert_close(pooled[r], want[r * bl:(r + 1) * bl], rtol=1e-5, atol=1e-6)
        g = torch.randn(cfg.global_batch, cfg.num_tables, cfg.dim, device="cuda")
        for r in range(world):
            models[r].sparse_backward_launch(g[r * bl:(r + 1) * bl])
        for r in range(world):
            models[r].sparse_backward_apply(batches[r][1])
        torch.cuda.synchronize()
        ref.embedding_bag_sgd(full_tables, full_idx, g, cfg.lr)
        got = torch.cat([m.tables for m in models])
        for r in range(world):
            heaps[r].check_status()
        torch.testing.assert_close(got, full_tables, rtol=1e-4, atol=1e-5)
    finally:
        for h in heaps:
            h.close()


def test_out_of_range_index_is_reported_not_faulted():
    from fuselink_b200.models.dlrm import DLRM, synthetic_batch
    from fuselink_b200.parallel.symm import SymmetricHeap
    cfg = _cfg(num_tables=2, global_batch=64)
    heaps = SymmetricHeap.emulated(1, 16 << 20)
    try:
        m = DLRM(cfg, heaps[0], 0, 1, device="cuda")
        _, idx, _ = synthetic_batch(cfg, 0, 1, "cuda", seed=0)
        idx[0, 3, 4] = cfg.rows + 17
        m.sparse_forward_launch(idx)
        m.sparse_forward_wait()
        torch.cuda.synchronize()
        with pytest.raises(RuntimeError, match="out of bounds"):
            heaps[0].check_status()
    finally:
        heaps[0].close()


def test_dlrm_train_step_matches_cpu_model():
    from fuselink_b200.models.dlrm import DLRM, synthetic_batch
    from fuselink_b200.parallel.symm import SymmetricHeap
    cfg = _cfg(num_tables=5, global_batch=256)
    heaps = SymmetricHeap.emulated(1, 16 << 20)
    try:
        gpu = DLRM(cfg, heaps[0], 0, 1, device="cuda", seed=2)
        cpu = DLRM(cfg, None, 0, 1, device="cpu", seed=2)
        cpu.tables.copy_(gpu.tables.cpu())
        cpu.bottom.load_state_dict({k: v.cpu() for k, v in gpu.bottom.state_dict().items()})
        cpu.top.load_state_dict({k: v.cpu() for k, v in gpu.top.state_dict().items()})
        og = torch.optim.SGD(gpu.dense_parameters(), lr=cfg.lr)
        oc = torch.optim.SGD(cpu.dense_parameters(), lr=cfg.lr)
        for step in range(3):
            d, i, l = synthetic_batch(cfg, 0, 1, "cuda", seed=10 + step)
            lg = gpu.train_step(d, i, l, og)
            lc = cpu.train_step(d.cpu(), i.cpu(), l.cpu(), oc)
            assert abs(float(lg) - float(lc)) < 2e-3, (step, float(lg), float(lc))
        torch.cuda.synchronize()
        heaps[0].check_status()
        torch.testing.assert_close(gpu.tables.cpu(), cpu.tables, rtol=1e-3, atol=1e-5)
    finally:
        heaps[0].close()
