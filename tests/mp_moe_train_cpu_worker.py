"""Worker of tests/test_kernel_model_cpu.py::test_moe_transformer_trains_between_processes: a tiny MoE transformer trained for a
few steps by real processes on a machine without a GPU -- experts spread over the ranks with the hottest one shadowed and
chosen again every step, everything else data parallel -- through the fused path of the MoE layer (device entry points
modelled on the host, shared-memory heap).  Checks what a training job relies on: the replicated parameters and the copies
of the shadowed experts stay identical on every rank, the loss is finite and falls."""
import dataclasses
import datetime
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import torch
import torch.distributed as dist


def same_everywhere(t, what):
    parts = [torch.empty_like(t) for _ in range(dist.get_world_size())]
    dist.all_gather(parts, t.contiguous())
    assert all(torch.equal(p, parts[0]) for p in parts), f"{what} differs between ranks"


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=120))
    import cpu_kernel_model
    from fuselink_b200.models.moe_transformer import MOE_ZOO, MoETransformer
    from fuselink_b200.parallel.symm import SymmetricHeap
    B, S = 2, 16
    cfg = dataclasses.replace(MOE_ZOO["tiny_moe"], shadow_experts=1)
    with cpu_kernel_model.installed(single_process=False, lock_path=os.environ["FL_MODEL_LOCK"]) as model:
        model.wait_limit_s = 30.0
        heap = SymmetricHeap.create(64 << 20, device=-1)
        net = MoETransformer(cfg, B * S, heap, rank, world, device="cpu", seed=3)      # bf16, as on the GPU: the fused path takes bf16 rows
        assert all(b.moe.ws is not None and len(b.moe.cfg.shadow) == 1 for b in net.blocks)
        opt = torch.optim.SGD(net.parameters(), lr=0.3)
        gen = torch.Generator().manual_seed(17 + rank)
        tokens = torch.randint(0, cfg.vocab, (B, S), generator=gen)
        labels = torch.roll(tokens, -1, 1)
        losses = []
        for step in range(4):
            losses.append(float(net.train_step(tokens, labels, opt)))          # the same batch every step: the loss must fall
            heap.check_status(f"step {step}")
            for b in net.blocks:
                b.moe.reshadow(tolerance=0.0)
            for i, b in enumerate(net.blocks):
                epr = b.moe.epr
                same_everywhere(b.moe.w2.data[epr:], f"copies of layer {i}")
                same_everywhere(b.wqkv.data, f"attention weights of layer {i}")
                same_everywhere(b.moe.router.data, f"router of layer {i}")
        assert all(l == l and l < 20 for l in losses) and losses[-1] < losses[0], losses
        dist.barrier()
        print(f"MOE-TRAIN-OK rank {rank} losses {[round(l, 3) for l in losses]}", flush=True)
        heap.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
