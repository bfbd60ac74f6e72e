"""Idleness monitor and path selector on the CPU: state transitions, leases, borrow rules, synthetic
Poisson traffic (mean 1 GB/s per path), multi-process sharing through POSIX shm, and lock-free stress."""
import os
import random
import subprocess
import sys
import threading
import time
import uuid

import pytest

from fuselink_b200 import C, have_native

pytestmark = pytest.mark.skipif(not have_native(), reason="native extension not built")

IDLE, BUSY, BORROWED, DEAD = 0, 1, 2, 3
TX, RX = 0, 1
US = 1000


def test_idle_busy_lease_expiry():
    m = C.monitor_open("", True, 8, 1, 160)
    t = 1_000_000
    assert C.monitor_status(m, TX, 3) == IDLE
    C.monitor_mark_active(m, TX, 3, t)
    assert C.monitor_status(m, TX, 3) == BUSY
    C.monitor_sweep(m, t + 100 * US)
    assert C.monitor_status(m, TX, 3) == BUSY          # inside the 160 us window
    C.monitor_sweep(m, t + 160 * US)
    assert C.monitor_status(m, TX, 3) == IDLE          # last_active + timeout <= now
    assert C.monitor_status(m, RX, 3) == IDLE          # directions are independent
    C.monitor_close(m, False)


def test_outstanding_bytes_keep_a_path_busy():
    m = C.monitor_open("", True, 4, 1, 160)
    t = 5_000_000
    C.monitor_post_bytes(m, TX, 1, 1 << 20, t)
    C.monitor_sweep(m, t + 10_000 * US)
    assert C.monitor_status(m, TX, 1) == BUSY and C.monitor_outstanding(m, TX, 1) == 1 << 20
    C.monitor_complete_bytes(m, TX, 1, 1 << 20, t + 10_001 * US)
    C.monitor_sweep(m, t + 10_100 * US)
    assert C.monitor_status(m, TX, 1) == BUSY          # completed 99 us ago
    C.monitor_sweep(m, t + 10_200 * US)
    assert C.monitor_status(m, TX, 1) == IDLE
    C.monitor_close(m, False)


def test_borrow_rules():
    m = C.monitor_open("", True, 4, 2, 160)            # 4 groups x 2 paths
    t = 1_000_000
    full = (1 << 8) - 1
    # never a path of the own group (group 1 = paths 2, 3)
    got = {C.monitor_borrow_idle(m, TX, 1, 2, full, t) for _ in range(6)}
    assert got == {4, 5, 6, 7, 0, 1}
    assert C.monitor_borrow_idle(m, TX, 1, 2, full, t) == -1      # everything else is borrowed
    assert C.monitor_status(m, TX, 4) == BORROWED
    # mask restricts candidates
    C.monitor_release(m, TX, 6)
    C.monitor_release(m, TX, 7)
    assert C.monitor_borrow_idle(m, TX, 1, 2, 1 << 7, t) == 7
    # a crashed borrower's lease expires by timestamp
    C.monitor_sweep(m, t + 1000 * US)
    assert C.monitor_status(m, TX, 4) == IDLE
    # dead paths are never handed out
    C.monitor_mark_dead(m, TX, 0, True)
    for _ in range(8):
        assert C.monitor_borrow_idle(m, TX, 1, 7, full, t + 2000 * US) != 0
    C.monitor_close(m, False)


def test_external_counters_feed_completion():
    import torch
    m = C.monitor_open("", True, 4, 1, 160)
    ctr = torch.zeros(4, dtype=torch.int64)                       # stands in for GPU-written pinned memory
    C.monitor_attach_counters(m, TX, ctr.data_ptr())
    t = 1_000_000
    C.monitor_post_bytes(m, TX, 2, 4096, t)
    ctr[2] = 4096
    C.monitor_sweep(m, t + 10 * US)
    assert C.monitor_outstanding(m, TX, 2) == 0 and C.monitor_status(m, TX, 2) == BUSY
    C.monitor_sweep(m, t + 400 * US)
    assert C.monitor_status(m, TX, 2) == IDLE
    C.monitor_attach_counters(m, TX, 0)
    C.monitor_close(m, False)


def test_poisson_traffic_and_selector():
    """Synthetic per-path byte counters: Poisson arrivals, mean 1 GB/s on the busy paths."""
    rng = random.Random(0)
    m = C.monitor_open("", True, 8, 1, 160)
    busy = [0, 1, 2]
    t = 10_000_000
    msg = 64 * 1024
    rate = 1e9 / msg                                              # messages per second for 1 GB/s
    nxt = {p: t + int(rng.expovariate(rate) * 1e9) for p in busy}
    end = t + 20_000 * US
    picks = []
    while t < end:
        t += 20 * US
        for p in busy:
            while nxt[p] <= t:
                C.monitor_post_bytes(m, TX, p, msg, nxt[p])
                C.monitor_complete_bytes(m, TX, p, msg, nxt[p] + 5 * US)
                nxt[p] += int(rng.expovariate(rate) * 1e9)
        C.monitor_sweep(m, t)
        if (t // (20 * US)) % 50 == 0:
            s = C.select_paths(m, 3, 1, 1 << 20, 512 * 1024, True, 0, 1, 64 << 20, len(picks), t)
            picks.append(s)
            for path, _, _ in s[1:]:
                C.monitor_release(m, TX, path)
    # mean inter-arrival is 65 us << 160 us, so busy paths are (almost) never idle; relays come from 3..7
    relay_paths = [p for s in picks for p, _, _ in s[1:]]
    assert relay_paths, "selector never used a relay although 5 paths were idle"
    assert sum(1 for p in relay_paths if p in busy) <= 0.05 * len(relay_paths)
    for s in picks:
        assert s[0][0] == 1 and sum(b for _, _, b in s) == 64 << 20
        assert all(off % (512 * 1024) == 0 for _, off, _ in s)
    for p in busy:
        assert 0.5 < C.monitor_bandwidth_gbs(m, TX, p) < 2.0, C.monitor_bandwidth_gbs(m, TX, p)
    assert C.monitor_bandwidth_gbs(m, TX, 5) == 0
    C.monitor_close(m, False)


def test_selector_answers_direct():
    m = C.monitor_open("", True, 8, 1, 160)
    now = C.monitor_now_ns()
    assert C.select_paths(m, 1, 1, 1 << 20, 4096, True, 0, 1, 1 << 30, 0, now) == [(1, 0, 1 << 30)]   # degree 1
    assert C.select_paths(m, 4, 1, 1 << 20, 4096, False, 0, 1, 1 << 30, 0, now) == [(1, 0, 1 << 30)]  # relays off
    assert C.select_paths(m, 4, 1, 1 << 20, 4096, True, 0, 1, 100_000, 0, now) == [(1, 0, 100_000)]   # too small
    for p in range(2, 8):
        C.monitor_mark_active(m, TX, p, now)
    assert len(C.select_paths(m, 4, 1, 1 << 20, 4096, True, 0, 1, 1 << 30, 0, now)) == 1             # nothing idle
    C.monitor_close(m, False)


def test_shared_table_between_processes():
    name = "/fl_test_" + uuid.uuid4().hex[:12]
    m = C.monitor_open(name, True, 8, 1, 160)
    code = (
        "import sys; sys.path.insert(0, %r)\n"
        "from fuselink_b200 import C\n"
        "m = C.monitor_open(%r, False, 8, 1, 160)\n"
        "p = C.monitor_borrow_idle(m, 0, 0, 0, 0xff, C.monitor_now_ns())\n"
        "print(p)\n" % (os.path.dirname(os.path.dirname(os.path.abspath(__file__))), name))
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=120)
    assert out.returncode == 0, out.stderr
    p = int(out.stdout.strip().splitlines()[-1])
    assert p == 1 and C.monitor_status(m, TX, 1) == BORROWED      # visible in this process
    C.monitor_close(m, True)
    with pytest.raises(RuntimeError):
        C.monitor_open(name, False, 8, 1, 160)                    # daemon gone -> clients are told


def test_lock_free_borrow_is_exclusive_under_contention():
    m = C.monitor_open("", True, 16, 1, 1_000_000)
    C.monitor_start(m, 40)
    held, lock, errors = set(), threading.Lock(), []

    def worker(group):
        for _ in range(3000):
            p = C.monitor_borrow_idle(m, TX, group, group, 0xffff, C.monitor_now_ns())
            if p < 0:
                continue
            with lock:
                if p in held:
                    errors.append(p)
                held.add(p)
            with lock:
                held.discard(p)
            C.monitor_release(m, TX, p)

    ths = [threading.Thread(target=worker, args=(g,)) for g in range(4)]
    [t.start() for t in ths]
    [t.join() for t in ths]
    C.monitor_stop(m)
    assert not errors, f"paths handed to two borrowers at once: {errors[:5]}"
    C.monitor_close(m, False)


def test_daemon_binary_creates_and_removes_table():
    exe = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "fuselink_b200", "lib", "fuselink-monitor")
    if not os.path.exists(exe):
        pytest.skip("daemon not built")
    name = "/fl_daemon_" + uuid.uuid4().hex[:10]
    p = subprocess.Popen([exe, "--shm", name, "--seconds", "1.0"], stdout=subprocess.PIPE, text=True)
    t0 = time.time()
    m = None
    while m is None and time.time() - t0 < 5:
        try:
            m = C.monitor_open(name, False, 8, 1, 160)
        except RuntimeError:
            time.sleep(0.02)
    assert m is not None
    C.monitor_mark_active(m, TX, 0, C.monitor_now_ns())
    time.sleep(0.05)
    assert C.monitor_status(m, TX, 0) == IDLE                     # the daemon's sweeper expired it
    C.monitor_close(m, False)
    assert p.wait(timeout=10) == 0


def test_daemon_sizes_its_table_from_the_machine():
    exe = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "fuselink_b200", "lib", "fuselink-monitor")
    if not os.path.exists(exe):
        pytest.skip("daemon not built")
    name = "/fl_daemon_" + uuid.uuid4().hex[:10]
    out = subprocess.run([exe, "--shm", name, "--groups", "auto", "--seconds", "0.2"], capture_output=True, text=True, timeout=30)
    assert out.returncode == 0
    want = 0
    for d in ("/sys/class/infiniband", "/proc/driver/nvidia/gpus"):
        if want == 0 and os.path.isdir(d):
            want = len([e for e in os.listdir(d) if not e.startswith(".")])
    assert f"{want or 8} paths" in out.stdout, out.stdout


def test_daemon_bench_mode_reports_the_decision_latency():
    """`fuselink-monitor --bench` times a selector decision and the table's calls with the sweeper running; a decision is
    a few atomics and two clock reads, far below the 160 us lease it has to fit into."""
    import json
    exe = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "fuselink_b200", "lib", "fuselink-monitor")
    if not os.path.exists(exe):
        pytest.skip("daemon not built")
    for threads in (1, 3):
        out = subprocess.run([exe, "--bench", "100000", "--threads", str(threads)], capture_output=True, text=True, timeout=60)
        assert out.returncode == 0, out.stderr
        r = json.loads(out.stdout.strip().splitlines()[-1])
        assert r["threads"] == threads and r["paths"] == 8
        assert r["decisions"] >= 100000 * threads
        for k in ("select_paths_ns", "borrow_release_ns", "mark_active_ns", "post_complete_bytes_ns"):
            assert 0 < r[k] < 50_000, (k, r)               # generous: a shared CI core, not a latency claim


def test_metrics_endpoint_serves_the_table():
    """The Prometheus endpoint reads the same table the selector writes: state, outstanding bytes and decisions."""
    import urllib.request
    from fuselink_b200.utils.metrics import MetricsServer, render
    m = C.monitor_open("", True, 4, 1, 160)
    t = C.monitor_now_ns()
    C.monitor_post_bytes(m, TX, 2, 12345, t)
    C.monitor_mark_dead(m, RX, 1, True)
    text = render(C, m, {"failovers": 3})
    assert 'fuselink_path_outstanding_bytes{dir="tx",path="2"} 12345' in text
    assert f'fuselink_path_state{{dir="rx",path="1"}} {DEAD}' in text
    assert f'fuselink_path_state{{dir="tx",path="2"}} {BUSY}' in text
    assert "fuselink_failovers 3" in text
    srv = MetricsServer(C, m, port=0)
    try:
        body = urllib.request.urlopen(f"http://127.0.0.1:{srv.port}/metrics", timeout=10).read().decode()
        assert 'fuselink_path_outstanding_bytes{dir="tx",path="2"} 12345' in body and "fuselink_borrow_decisions_total" in body
        with pytest.raises(Exception):
            urllib.request.urlopen(f"http://127.0.0.1:{srv.port}/nope", timeout=10)
    finally:
        srv.close()
        C.monitor_close(m, False)


def test_selector_plans_partition_the_transfer_for_any_parameters():
    """Property test: whatever the size, degree, step, minimum stripe, alignment and set of busy paths, the stripes cover
    [0, bytes) exactly once, stripe 0 is the direct path, relay stripes start on the alignment and respect the minimum
    size, no relay is the source, the destination, a busy path or used twice."""
    hyp = pytest.importorskip("hypothesis")
    st = hyp.strategies

    @hyp.settings(max_examples=200, deadline=None)
    @hyp.given(nbytes=st.integers(0, 1 << 34), degree=st.integers(1, 8), step=st.integers(1, 4),
               min_stripe=st.sampled_from([4096, 1 << 16, 1 << 20, 1 << 24]), align=st.sampled_from([16, 256, 4096, 1 << 19]),
               src=st.integers(0, 7), dst=st.integers(0, 7), busy=st.sets(st.integers(0, 7)), index=st.integers(0, 1000))
    def check(nbytes, degree, step, min_stripe, align, src, dst, busy, index):
        hyp.assume(src != dst)
        m = C.monitor_open("", True, 8, 1, 160)
        try:
            now = C.monitor_now_ns()
            for p in busy:
                C.monitor_mark_active(m, TX, p, now)
            plan = C.select_paths(m, degree, step, min_stripe, align, True, src, dst, nbytes, index, now)
            assert 1 <= len(plan) <= degree
            assert plan[0][0] == dst
            pieces = sorted((off, n) for _, off, n in plan)
            pos = 0
            for off, n in pieces:
                assert off == pos
                pos += n
            assert pos == nbytes
            relays = [p for p, _, _ in plan[1:]]
            assert len(set(relays)) == len(relays)
            for p, off, n in plan[1:]:
                assert p not in (src, dst) and p not in busy
                assert off % align == 0 and n >= min_stripe
        finally:
            C.monitor_close(m, False)

    check()


def test_claim_is_exclusive_and_lapses_like_a_lease():
    m = C.monitor_open("", True, 4, 1, 160)
    t = 2_000_000
    assert C.monitor_claim(m, RX, 0, 111, t) == 1                    # idle -> held by owner 111
    assert C.monitor_status(m, RX, 0) == BORROWED
    assert C.monitor_claim(m, RX, 0, 111, t + 10 * US) == 1          # the holder may claim again
    assert C.monitor_claim(m, RX, 0, 222, t + 20 * US) == 0          # anybody else may not
    assert C.monitor_borrow_idle(m, RX, 1, 3, (1 << 64) - 1, t + 20 * US) != 0   # and it is not handed out as idle either
    C.monitor_sweep(m, t + 10 * US + 160 * US)
    assert C.monitor_status(m, RX, 0) == IDLE                        # nothing outstanding, no stamp for 160 us
    assert C.monitor_claim(m, RX, 0, 222, t + 400 * US) == 1
    C.monitor_mark_active(m, RX, 1, t)
    assert C.monitor_claim(m, RX, 1, 111, t + US) == 0               # busy with somebody's traffic
    C.monitor_close(m, False)


def test_plugin_counters_are_readable_from_python():
    from fuselink_b200.utils.metrics import plugin_counters, render
    c = plugin_counters()
    assert set(c) >= {"plugin_decisions", "plugin_fallbacks", "plugin_failovers", "plugin_direct_bytes", "plugin_rdma_pieces"}
    assert all(isinstance(v, int) and v >= 0 for v in c.values())
    m = C.monitor_open("", True, 2, 1, 160)
    try:
        assert "fuselink_plugin_failovers 0" in render(C, m, c)
    finally:
        C.monitor_close(m, False)
