"""Worker of tests/test_kernel_model_cpu.py::test_dlrm_fused_step_between_processes: the table-wise sharded DLRM step
between real processes on a machine without a GPU.  The fused path (pooled vectors stored into the sample owners' buffers,
gradients read back from them, SGD on the tables inside the backward entry point, dense gradients all-reduced in one
bucket while the sparse backward runs) goes through the host model of the embedding-bag entry points over a shared-memory
heap; the oracle is the same model's plain-PyTorch path over gloo, from the same seed."""
import datetime
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import torch
import torch.distributed as dist


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=120))
    import cpu_kernel_model
    from fuselink_b200.models.dlrm import DLRM, DLRMConfig, synthetic_batch
    from fuselink_b200.parallel.symm import SymmetricHeap
    cfg = DLRMConfig(num_tables=7, rows=200, dim=128, pooling=5, global_batch=24 * world, lr=0.1)
    with cpu_kernel_model.installed(single_process=False) as model:
        model.wait_limit_s = 30.0
        heap = SymmetricHeap.create(16 << 20, device=-1)
        fused = DLRM(cfg, heap, rank, world, device="cpu", seed=5)
        plain = DLRM(cfg, None, rank, world, device="cpu", seed=5)
        assert torch.equal(fused.tables, plain.tables)
        of, op = torch.optim.SGD(fused.dense_parameters(), lr=cfg.lr), torch.optim.SGD(plain.dense_parameters(), lr=cfg.lr)
        for step in range(3):
            d, i, l = synthetic_batch(cfg, rank, world, "cpu", seed=step)
            lf = fused.train_step(d, i, l, of)
            heap.check_status(f"step {step}")
            lp = plain.train_step(d, i, l, op)
            assert abs(float(lf) - float(lp)) < 1e-5, (step, float(lf), float(lp))
            assert torch.allclose(fused.tables, plain.tables, atol=1e-6), f"tables differ after step {step}"
            for a, b in zip(fused.dense_parameters(), plain.dense_parameters()):
                assert torch.allclose(a, b, atol=1e-6), f"dense weights differ after step {step}"
        assert fused.launches > 0
        dist.barrier()
        print(f"DLRM-MP-OK rank {rank}", flush=True)
        heap.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
