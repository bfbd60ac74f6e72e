"""Failure detection without a GPU fault: every failure is made on the host (a rank that exits between steps,
a dead path in the monitor, a process group whose collective times out)."""
import datetime
import os
import socket
import time

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from fuselink_b200 import C, have_native


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _leaver(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=3))
    t = torch.ones(4)
    dist.all_reduce(t)                      # step 0: everyone is here
    if rank == 1:
        dist.destroy_process_group()        # leaves BETWEEN steps, nothing in flight
        return
    t0 = time.time()
    try:
        dist.all_reduce(t)                  # step 1: the survivor's collective must end with an error, not hang
        q.put(("no-error", time.time() - t0))
    except Exception as e:                  # noqa: BLE001
        q.put(("error", time.time() - t0, type(e).__name__))


def test_rank_leaving_between_steps_is_detected_by_timeout():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_leaver, args=(r, 2, _free_port() if r == 0 else 0, q)) for r in range(2)]
    port = _free_port()
    procs = [ctx.Process(target=_leaver, args=(r, 2, port, q)) for r in range(2)]
    [p.start() for p in procs]
    res = q.get(timeout=60)
    [p.join(timeout=30) for p in procs]
    assert res[0] == "error" and res[1] < 30, res


@pytest.mark.skipif(not have_native(), reason="native extension not built")
def test_dead_path_is_routed_around_and_recovers():
    from fuselink_b200.parallel.selector import PathSelector
    os.environ["NCCL_FUSELINK_DEGREE"] = "3"
    os.environ["FUSELINK_MIN_STRIPE_BYTES"] = str(1 << 20)
    try:
        sel = PathSelector(4)
        plan = sel.plan(0, 1, 64 << 20)
        assert {p for p, _, _ in plan} == {1, 2, 3}
        sel.complete(0, 1, 64 << 20, plan)
        sel.mark_dead(2)
        for _ in range(5):
            plan = sel.plan(0, 1, 64 << 20)
            assert 2 not in {p for p, _, _ in plan}, "a dead relay must never be selected"
            assert sum(b for _, _, b in plan) == 64 << 20
            sel.complete(0, 1, 64 << 20, plan)
        sel.mark_dead(2, False)
        time.sleep(0.01)
        seen = set()
        for _ in range(6):
            plan = sel.plan(0, 1, 64 << 20)
            seen |= {p for p, _, _ in plan}
            sel.complete(0, 1, 64 << 20, plan)
        assert 2 in seen, "a revived path is used again"
        sel.close()
    finally:
        os.environ.pop("NCCL_FUSELINK_DEGREE")
        os.environ.pop("FUSELINK_MIN_STRIPE_BYTES")


@pytest.mark.skipif(not have_native(), reason="native extension not built")
def test_crashed_borrower_releases_its_lease_by_timeout():
    m = C.monitor_open("", True, 4, 1, 160)
    t = C.monitor_now_ns()
    p = C.monitor_borrow_idle(m, 0, 0, 0, 0xF, t)
    assert p >= 0 and C.monitor_status(m, 0, p) == 2
    # the borrower "crashes": no release, no stamps.  One lease period later the path is idle again.
    C.monitor_sweep(m, t + 161_000)
    assert C.monitor_status(m, 0, p) == 0
    C.monitor_close(m, False)


def _hb_worker(rank, world, port, q, mode):
    from fuselink_b200.parallel.health import Heartbeat, PeerLost, renumber
    store = dist.TCPStore("127.0.0.1", port, world, is_master=(rank == 0), timeout=datetime.timedelta(seconds=20))
    hb = Heartbeat(store, rank, world, interval_s=0.05, timeout_s=0.6)
    assert hb.wait_all_seen(20)
    hb.check()                                     # step 0: everybody is here
    store.set(f"step0/{rank}", "1")                # ... and nobody goes before everybody has finished that step
    store.wait([f"step0/{r}" for r in range(world)], datetime.timedelta(seconds=60))
    if rank == world - 1:
        if mode == "crash":
            os._exit(0)                            # dies between steps without a word
        hb.leave()                                 # or says goodbye
        time.sleep(2.0)                            # keep the process (not the heartbeat) around
        return
    t0 = time.time()
    err = None
    while time.time() - t0 < 15 and err is None:
        try:
            hb.check()                             # what a training loop calls before the next launch
            time.sleep(0.05)
        except PeerLost as e:
            err = e
    surv = hb.survivors()
    q.put((rank, None if err is None else (err.lost, err.left), time.time() - t0, surv, renumber(surv, rank)))
    hb.close()
    store.set(f"done/{rank}", "1")
    if rank == 0:                                  # the store's host outlives the others' last reads
        t1 = time.time()
        while time.time() - t1 < 20 and not all(store.check([f"done/{r}"]) for r in surv):
            time.sleep(0.05)
        time.sleep(0.2)


@pytest.mark.parametrize("mode", ["crash", "leave"])
def test_heartbeat_detects_a_lost_or_leaving_rank_before_the_next_launch(mode):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    world = 3
    procs = [ctx.Process(target=_hb_worker, args=(r, world, port, q, mode)) for r in range(world)]
    [p.start() for p in procs]
    got = sorted(q.get(timeout=120) for _ in range(world - 1))
    [p.join(timeout=30) for p in procs]
    for rank, err, dt, surv, (new_rank, new_world) in got:
        assert err is not None, "the loss went unnoticed"
        lost, left = err
        assert (lost, left) == (([2], []) if mode == "crash" else ([], [2]))
        assert dt < (10.0 if mode == "crash" else 6.0)           # lease expiry vs an explicit goodbye (generous: loaded CI hosts)
        assert surv == [0, 1] and (new_rank, new_world) == (rank, 2)


def test_rank_leaves_between_steps_and_the_others_carry_on():
    """Three processes over a heap they really share (memfd regions, descriptors over SCM_RIGHTS), the device entry
    points replaced by their host model: an all-to-all with everybody, the last rank leaves cleanly, the other two learn
    of it from the heartbeat, run a ring of puts among themselves, and a wait on the leaver runs out into the status word."""
    import subprocess
    import sys
    here = os.path.dirname(os.path.abspath(__file__))
    port = _free_port()
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=3", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(here, "mp_leave_cpu_worker.py")]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=180)
    assert out.stdout.count("LEAVE-OK") == 2, out.stdout[-3000:] + out.stderr[-3000:]
