"""Device-side waits are bounded: a wait on a flag that nothing ever sets gives up after its limit, records a status code
the host can read, and leaves the CUDA context usable.  No fault, trap or endless loop is involved."""
import time

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_flag_wait_runs_out_and_reports_status():
    from fuselink_b200 import C
    from fuselink_b200.parallel.symm import SymmetricHeap
    heaps = SymmetricHeap.emulated(2, 8 << 20)
    try:
        h = heaps[0]
        slot = h.signal_slots("never-set", 1)
        t0 = time.time()
        C.wait_flags([(h.sig_addr(slot), 1)], h.status_addr, 50)      # 50 ms limit
        torch.cuda.synchronize()
        assert time.time() - t0 < 5.0
        st = h.status().cpu().tolist()
        assert st[0] == 1 and st[1] == 700, st                          # kTimeoutFlag, recorded by wait #0
        with pytest.raises(RuntimeError, match="flag wait timed out"):
            h.check_status("timeout test")
        assert h.status()[0].item() == 0                                # reading the status clears it
        # the context is alive and the same flag, once set, satisfies a new wait immediately
        h.signals()[slot] = 1
        C.wait_flags([(h.sig_addr(slot), 1)], h.status_addr, 50)
        x = torch.ones(1024, device="cuda").sum().item()
        torch.cuda.synchronize()
        assert x == 1024 and h.status()[0].item() == 0
    finally:
        for hh in heaps:
            hh.close()


def test_put_kernel_feeds_monitor_counters():
    """The put kernel adds the bytes of every finished chunk to a pinned host counter that the monitor's sweeper folds
    into the path's completed bytes (device-side completion counters -> lock-free host thread)."""
    from fuselink_b200 import C
    from fuselink_b200.ops.comm import Channel
    from fuselink_b200.parallel.selector import PathSelector
    from fuselink_b200.parallel.symm import SymmetricHeap
    heaps = SymmetricHeap.emulated(2, 32 << 20)
    sel = PathSelector(2)
    try:
        ch = Channel(heaps[0], "ctr")
        ctr = ch.attach_counters(sel)
        dst = heaps[0].alloc_tensor([4 << 20], torch.uint8)
        src = torch.randint(0, 255, (4 << 20,), dtype=torch.uint8, device="cuda")
        C.monitor_post_bytes(sel.mon, 0, 1, 4 << 20, C.monitor_now_ns())
        ch.put(src, 1, dst.offset)
        torch.cuda.synchronize()
        assert int(ctr[1]) == 4 << 20 and int(ctr[0]) == 0
        time.sleep(0.01)                                  # a few sweeps of the monitor thread
        assert C.monitor_outstanding(sel.mon, 0, 1) == 0
    finally:
        sel.close()
        for h in heaps:
            h.close()
