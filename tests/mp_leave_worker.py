"""Worker of tests/test_multigpu.py::test_rank_leaving_between_steps_on_gpus: one process per GPU, NVLS off, plain
peer stores.  The last rank leaves BETWEEN steps with nothing in flight; the others learn of it on the host through the
heartbeat before they launch anything that would wait for it, and keep working among themselves on the same heap."""
import datetime
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist


def main():
    rank, local, world = int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=30))
    from fuselink_b200.ops.comm import Channel, all_to_all, barrier
    from fuselink_b200.parallel.health import Heartbeat, PeerLost
    from fuselink_b200.parallel.symm import SymmetricHeap

    store = dist.TCPStore("127.0.0.1", int(os.environ["MASTER_PORT"]) + 7, world, is_master=(rank == 0),
                          timeout=datetime.timedelta(seconds=30))
    hb = Heartbeat(store, rank, world, interval_s=0.05, timeout_s=1.0)
    assert hb.wait_all_seen(30)
    heap = SymmetricHeap.create(64 << 20, device=local)
    ch = Channel(heap, "leave", engine="ldst")
    per = 50_000
    recv = heap.alloc_tensor([world, per], torch.float32)
    ring = heap.alloc_tensor([1 << 20], torch.uint8)

    # ---- step 0: everybody takes part ---------------------------------------------------------------------
    hb.check()
    send = torch.full((world, per), float(rank), device=dev)
    all_to_all(ch, send, recv)
    torch.cuda.synchronize()
    want = torch.arange(world, device=dev, dtype=torch.float32).unsqueeze(1).expand(world, per)
    assert torch.equal(recv.local, want)
    barrier(heap, "leave-b0")
    torch.cuda.synchronize()
    heap.check_status("step 0")
    dist.barrier()

    # ---- between steps: the last rank goes --------------------------------------------------------------------
    if rank == world - 1:
        hb.leave()
        heap.close()
        time.sleep(3.0)
        os._exit(0)

    # ---- the others notice on the host, before launching anything that waits for the leaver -------------------
    lost = None
    t0 = time.time()
    while lost is None and time.time() - t0 < 20:
        try:
            hb.check()
            time.sleep(0.05)
        except PeerLost as e:
            lost = e
    assert lost is not None and lost.left == [world - 1] and not lost.lost, lost
    surv = hb.survivors()
    assert surv == list(range(world - 1)), surv
    # step 1 among the survivors only: a ring of puts on the same heap (no kernel names the leaver)
    n = len(surv)
    if n > 1:
        nxt, prv = surv[(surv.index(rank) + 1) % n], surv[(surv.index(rank) - 1) % n]
        src = torch.full((1 << 20,), rank + 1, dtype=torch.uint8, device=dev)
        ch2 = Channel(heap, "leave-ring", engine="ldst")
        ch2.put(src, nxt, ring.offset)
        ch2.expect(prv, 1 << 20)
        ch2.wait([prv])
        torch.cuda.synchronize()
        assert bool((ring.local == prv + 1).all())
    heap.check_status("step 1")
    print(f"LEAVE-OK rank {rank} noticed after {time.time() - t0:.2f} s", flush=True)
    hb.close()
    heap.close()
    os._exit(0)          # the default process group still names the leaver: no collective teardown


if __name__ == "__main__":
    main()
