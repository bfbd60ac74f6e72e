"""Worker of tests/test_fault_cpu.py::test_rank_leaves_between_steps_and_the_others_carry_on: the scenario of
tests/mp_leave_worker.py on a machine without a GPU.  One process per rank over gloo; the symmetric heap is memfd-backed
host memory that the processes really share (descriptors passed over SCM_RIGHTS); the copy / flag / barrier entry points
are the functional model of tests/cpu_kernel_model.py, whose waits are real and bounded.  The last rank leaves BETWEEN
steps with nothing in flight; the others learn of it on the host through the heartbeat before they start anything that
would wait for it, keep working among themselves on the same heap, and a wait on the leaver -- started on purpose at the
end -- runs out and is reported through the status word instead of hanging."""
import datetime
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import torch
import torch.distributed as dist


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=60))
    import cpu_kernel_model
    from fuselink_b200.ops.comm import Channel, all_to_all, barrier
    from fuselink_b200.parallel.health import Heartbeat, PeerLost, renumber
    from fuselink_b200.parallel.symm import SymmetricHeap

    store = dist.TCPStore("127.0.0.1", int(os.environ["MASTER_PORT"]) + 7, world, is_master=(rank == 0),
                          timeout=datetime.timedelta(seconds=60))
    hb = Heartbeat(store, rank, world, interval_s=0.05, timeout_s=1.0)
    assert hb.wait_all_seen(30)
    with cpu_kernel_model.installed(single_process=False) as model:
        model.wait_limit_s = 1.0
        heap = SymmetricHeap.create(16 << 20, device=-1)
        assert heap.world == world and len(set(heap.base)) == world
        ch = Channel(heap, "leave", engine="ldst")
        per = 5_000
        recv = heap.alloc_tensor([world, per], torch.float32)
        ring = heap.alloc_tensor([1 << 16], torch.uint8)

        # ---- step 0: everybody takes part ------------------------------------------------------------------
        hb.check()
        send = torch.full((world, per), float(rank))
        all_to_all(ch, send, recv)
        want = torch.arange(world, dtype=torch.float32).unsqueeze(1).expand(world, per)
        assert torch.equal(recv.local, want)
        barrier(heap, "leave-b0")
        heap.check_status("step 0")
        dist.barrier()

        # ---- between steps: the last rank goes ------------------------------------------------------------
        if rank == world - 1:
            hb.leave()
            heap.close()
            time.sleep(2.0)
            os._exit(0)

        # ---- the others notice on the host, before starting anything that waits for the leaver ------------
        lost, t0 = None, time.time()
        while lost is None and time.time() - t0 < 20:
            try:
                hb.check()
                time.sleep(0.05)
            except PeerLost as e:
                lost = e
        assert lost is not None and lost.left == [world - 1] and not lost.lost, lost
        surv = hb.survivors()
        assert surv == list(range(world - 1)) and renumber(surv, rank) == (rank, world - 1)
        n = len(surv)
        if n > 1:                                        # step 1: a ring of puts among the survivors, same heap
            nxt, prv = surv[(surv.index(rank) + 1) % n], surv[(surv.index(rank) - 1) % n]
            src = torch.full((1 << 16,), rank + 1, dtype=torch.uint8)
            ch2 = Channel(heap, "leave-ring", engine="ldst")
            ch2.put(src, nxt, ring.offset)
            ch2.expect(prv, 1 << 16)
            ch2.wait([prv])
            assert bool((ring.local == prv + 1).all())
        heap.check_status("step 1")
        # what would have happened without the heartbeat: a wait for the leaver gives up after its limit and says so
        ch.expect(world - 1, 4 * per)
        t1 = time.time()
        ch.wait([world - 1])
        try:
            heap.check_status("wait for the leaver")
            raise AssertionError("the wait for a rank that left must be reported")
        except RuntimeError as e:
            assert "flag wait timed out" in str(e) and 0.9 < time.time() - t1 < 5.0, (str(e), time.time() - t1)
        print(f"LEAVE-OK rank {rank} noticed after {time.time() - t0:.2f} s", flush=True)
        hb.close()
        heap.close()
    os._exit(0)          # the default process group still names the leaver: no collective teardown


if __name__ == "__main__":
    main()
