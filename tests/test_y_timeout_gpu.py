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
