"""Worker of tests/test_kernel_model_cpu.py::test_striped_transfer_over_relays_between_processes: one rank-0 -> rank-1
transfer striped over the direct path and two relay ranks, four real processes on a machine without a GPU.  The stripes
come from the path selector (monitor table, degree 3); the copy / flag entry points are the host model over a shared-memory
heap, so the relays really wait for the source's per-chunk flags and the destination for its arrival counter."""
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
    from fuselink_b200.ops.comm import StripedP2P
    from fuselink_b200.parallel.selector import PathSelector
    from fuselink_b200.parallel.symm import SymmetricHeap
    with cpu_kernel_model.installed(single_process=False, lock_path=os.environ["FL_MODEL_LOCK"]) as model:
        model.wait_limit_s = 30.0
        heap = SymmetricHeap.create(64 << 20, device=-1)
        nbytes = (6 << 20) + 4096
        dst = heap.alloc_tensor([nbytes], torch.uint8)
        dsts = [heap.alloc_tensor([nbytes], torch.uint8) for _ in range(4)]
        striped = StripedP2P(heap, "t", 8 << 20)
        sel = PathSelector(world)                                     # every rank plans on its own table: same inputs, same plan
        # four transfers back to back, nothing between them: the relays' staging halves are reused, and what keeps the source
        # from overwriting a stripe a relay is still forwarding is the credit it reads from the relay
        plan = sel.plan(0, 1, nbytes)
        for it in range(4):
            src = torch.randint(0, 255, (nbytes,), dtype=torch.uint8, generator=torch.Generator().manual_seed(100 + it)) if rank == 0 else None
            striped.transfer(0, 1, src, dsts[it], nbytes, plan)
        sel.complete(0, 1, nbytes, plan)
        heap.check_status("back to back")
        if rank == 1:
            for it in range(4):
                want = torch.randint(0, 255, (nbytes,), dtype=torch.uint8, generator=torch.Generator().manual_seed(100 + it))
                assert torch.equal(dsts[it].local, want), f"back-to-back transfer {it} arrived damaged"
        dist.barrier()
        for it in range(3):
            stripes = sel.plan(0, 1, nbytes)
            paths = [p for p, _, _ in stripes]
            assert paths[0] == 1 and len(stripes) == 3 and set(paths[1:]) <= {2, 3}, stripes
            assert sum(b for _, _, b in stripes) == nbytes and all(o % 16 == 0 for _, o, _ in stripes)
            src = None
            if rank == 0:
                src = torch.randint(0, 255, (nbytes,), dtype=torch.uint8, generator=torch.Generator().manual_seed(it))
            striped.transfer(0, 1, src, dst, nbytes, stripes)
            sel.complete(0, 1, nbytes, stripes)
            heap.check_status(f"transfer {it}")
            if rank == 1:
                want = torch.randint(0, 255, (nbytes,), dtype=torch.uint8, generator=torch.Generator().manual_seed(it))
                assert torch.equal(dst.local, want), f"transfer {it} arrived damaged"
            dist.barrier()                                            # the destination buffer is reused
        assert sel.relay_answers == 4
        # a relay is declared dead (every rank hears of it on the host): the next plans leave it out and the transfer still arrives
        sel.mark_dead(2)
        for it in range(3, 5):
            stripes = sel.plan(0, 1, nbytes)
            paths = [p for p, _, _ in stripes]
            assert paths[0] == 1 and 2 not in paths and sum(b for _, _, b in stripes) == nbytes, stripes
            src = torch.randint(0, 255, (nbytes,), dtype=torch.uint8, generator=torch.Generator().manual_seed(it)) if rank == 0 else None
            striped.transfer(0, 1, src, dst, nbytes, stripes)
            sel.complete(0, 1, nbytes, stripes)
            heap.check_status(f"transfer {it} without relay 2")
            if rank == 1:
                want = torch.randint(0, 255, (nbytes,), dtype=torch.uint8, generator=torch.Generator().manual_seed(it))
                assert torch.equal(dst.local, want), f"transfer {it} arrived damaged"
            dist.barrier()
        sel.mark_dead(3)
        assert [p for p, _, _ in sel.plan(0, 1, nbytes)] == [1], "with no relay left the answer is the direct path"
        sel.close()
        print(f"RELAY-MP-OK rank {rank}", flush=True)
        heap.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
