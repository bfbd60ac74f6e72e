"""ncclNet plugin over the TCP transport, driven by two processes through the plugin's function table
(no NCCL, no GPU, no RDMA): bitwise transfer of {4 KB, 1 MB, 64 MB} fp32 messages in 512 KB chunks with 8
requests in flight, every ABI version, multi-path striping, and host-injected failures."""
import ctypes
import os
import subprocess
import sys
import tempfile

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB = os.path.join(ROOT, "fuselink_b200", "lib")
PLUGIN = os.path.join(LIB, "libnccl-net-fuselink.so")
HARNESS = os.path.join(LIB, "fl_net_harness")


@pytest.fixture(scope="module", autouse=True)
def _built():
    if not (os.path.exists(PLUGIN) and os.path.exists(HARNESS)):
        sys.path.insert(0, ROOT)
        from fuselink_b200 import build
        build.build_all()
    assert os.path.exists(PLUGIN) and os.path.exists(HARNESS)


def _pair(sizes, extra_send=(), extra_recv=(), env=None, common=(), timeout=120, env_send=None, env_recv=None):
    with tempfile.TemporaryDirectory() as d:
        hf = os.path.join(d, "handle")
        e = dict(os.environ, NCCL_SOCKET_IFNAME="lo", **(env or {}))
        sz = [str(s) for s in sizes]
        rx = subprocess.Popen([HARNESS, PLUGIN, "recv", hf, *common, *extra_recv, *sz], env=dict(e, **(env_recv or {})), stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
        tx = subprocess.Popen([HARNESS, PLUGIN, "send", hf, *common, *extra_send, *sz], env=dict(e, **(env_send or {})), stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
        try:
            txo, txe = tx.communicate(timeout=timeout)
            rxo, rxe = rx.communicate(timeout=timeout)
        finally:
            for p in (rx, tx):
                if p.poll() is None:
                    p.kill()
        return (tx.returncode, txo, txe), (rx.returncode, rxo, rxe)


@pytest.mark.parametrize("abi", [6, 7, 8])
def test_bitwise_transfer_reference_config(abi):
    tx, rx = _pair([4096, 1 << 20, 64 << 20], common=["--abi", str(abi), "--chunk", "524288", "--inflight", "8", "--seed", "0"])
    assert tx[0] == 0, tx
    assert rx[0] == 0, rx
    assert "OK received" in rx[1]


def test_odd_sizes_and_zero_length():
    tx, rx = _pair([0, 1, 3, 4097, 524288, 524289, 1234567], common=["--chunk", "65536"])
    assert tx[0] == 0 and rx[0] == 0, (tx, rx)


def test_striping_over_virtual_nics():
    env = {"NCCL_FUSELINK_DEGREE": "4", "NCCL_FUSELINK_STEP": "1", "FUSELINK_TCP_NDEV": "4", "FUSELINK_MIN_STRIPE_BYTES": "4096"}
    tx, rx = _pair([1 << 20, 8 << 20, 100_000], env=env)
    assert tx[0] == 0 and rx[0] == 0, (tx, rx)


def test_four_channels_side_by_side_spread_over_nics():
    """The reference's bandwidth configuration: 4 channels per peer, 512 KiB chunks, 8 steps in flight each
    (NCCL_NCHANNELS_PER_NET_PEER=4).  Chunk c travels on channel c % 4; every channel picks its NIC through the monitor."""
    env = {"FUSELINK_TCP_NDEV": "8", "NCCL_FUSELINK_DEGREE": "2", "FUSELINK_MIN_STRIPE_BYTES": "65536"}
    tx, rx = _pair([64 << 20, 1 << 20, 3], common=["--channels", "4", "--chunk", "524288", "--inflight", "8"], env=env)
    assert tx[0] == 0 and rx[0] == 0, (tx, rx)
    line = [l for l in rx[1].splitlines() if l.startswith("SELECTOR")][0].split()
    assert int(line[2]) >= 4            # at least one path decision per channel


def test_monitor_off_uses_channel_modulo():
    tx, rx = _pair([1 << 20], env={"FUSELINK_MONITOR": "0"})
    assert tx[0] == 0 and rx[0] == 0, (tx, rx)


def test_sender_death_is_reported_not_hung():
    """A sender that exits mid-transfer must surface as an error on the receiver (host-side fault)."""
    tx, rx = _pair([32 << 20], extra_send=["--die-after-chunks", "5"], extra_recv=["--expect-error"],
                   env={"FUSELINK_NET_TIMEOUT_MS": "3000"}, timeout=60)
    assert tx[0] == 9
    assert rx[0] == 0 and "EXPECTED-ERROR" in rx[1], rx


def test_link_failure_is_survived_by_moving_stripes_to_another_device():
    """A data socket breaks in the middle of a stripe: the sender marks the device dead and sends the stripe again, from
    its first byte, on the next device; the receiver drops the half stripe and the transfer completes bit for bit."""
    env = {"FUSELINK_FAULT_CLOSE_AFTER_BYTES": str(3 << 20), "FUSELINK_TCP_NDEV": "4", "NCCL_FUSELINK_DEGREE": "2",
           "FUSELINK_MIN_STRIPE_BYTES": "65536", "FUSELINK_NET_TIMEOUT_MS": "5000"}
    tx, rx = _pair([16 << 20, 4 << 20, 5], env=env, common=["--chunk", "524288", "--inflight", "8"], timeout=90)
    assert tx[0] == 0 and rx[0] == 0, (tx, rx)
    assert "FAILOVERS" in tx[1] and "lost (injected link failure)" in tx[2], tx


def test_injected_link_failure_marks_path_dead():
    tx, rx = _pair([16 << 20], extra_recv=["--expect-error"], env={"FUSELINK_FAULT_CLOSE_AFTER_BYTES": str(3 << 20), "FUSELINK_NET_TIMEOUT_MS": "3000",
                                                                   "FUSELINK_FAILOVER": "0"}, timeout=60)
    assert tx[0] != 0            # the sender reports the broken link
    assert rx[0] == 0 and "EXPECTED-ERROR" in rx[1], rx


def test_stalled_peer_times_out():
    """Receiver posts, the peer connects and then never sends: the request fails after
    FUSELINK_NET_TIMEOUT_MS instead of spinning forever."""
    import socket
    import struct
    import time
    with tempfile.TemporaryDirectory() as d:
        hf = os.path.join(d, "handle")
        e = dict(os.environ, NCCL_SOCKET_IFNAME="lo", NCCL_SOCKET_FAMILY="AF_INET", FUSELINK_NET_TIMEOUT_MS="500")
        rx = subprocess.Popen([HARNESS, PLUGIN, "recv", hf, "--expect-error", "65536"], env=e, stdout=subprocess.PIPE,
                              stderr=subprocess.PIPE, text=True)
        socks = []
        try:
            t0 = time.time()
            while not os.path.exists(hf):
                assert time.time() - t0 < 20
                time.sleep(0.01)
            h = open(hf, "rb").read()
            port = struct.unpack("!H", h[10:12])[0]
            ndev = struct.unpack("i", h[40:44])[0]
            # raw sockets with valid hellos so accept() completes; then stay silent
            for i in range(1 + ndev):
                s = socket.create_connection(("127.0.0.1", port))
                s.sendall(struct.pack("<QQiiii", 0x464c4e4b48454c4f, 0x1234, 0 if i == 0 else 1, -1 if i == 0 else i - 1, 0, ndev))
                socks.append(s)
            out, err = rx.communicate(timeout=30)
        finally:
            for s in socks:
                s.close()
            if rx.poll() is None:
                rx.kill()
        assert rx.returncode == 0 and "EXPECTED-ERROR" in out, (out, err)


def test_one_thread_per_channel():
    """NCCL drives the plugin from one proxy thread per device: four threads, each with its own connection, move every
    message concurrently through the shared selector and monitor."""
    env = {"FUSELINK_TCP_NDEV": "4", "NCCL_FUSELINK_DEGREE": "2", "FUSELINK_MIN_STRIPE_BYTES": "65536"}
    tx, rx = _pair([8 << 20, 4097, 0], common=["--channels", "4", "--threads", "--chunk", "262144", "--inflight", "8"], env=env)
    assert tx[0] == 0 and rx[0] == 0, (tx, rx)
    assert f"OK received {4 * ((8 << 20) + 4097)} bytes" in rx[1]


def test_device_buffers_are_adopted_rehomed_and_staged():
    """regMr on a "GPU" buffer (cuMem layer on its memfd stand-in): the buffer is adopted, re-homed onto the relay GPU
    (owner + channel) % nGPUs with its contents kept, and the bytes still arrive intact through the staging path."""
    env = {"FUSELINK_CUDA_PTRS": "1", "FUSELINK_VMM_FAKE": "1", "FUSELINK_VMM_FAKE_NGPUS": "8", "FL_HARNESS_VERBOSE": "1",
           "FUSELINK_NVL": "0"}
    tx, rx = _pair([3 << 20, 70000], env=env, common=["--device-buffers", "--dev", "2", "--chunk", "524288"],
                   extra_recv=["--channel", "3"], extra_send=[])
    assert tx[0] == 0 and rx[0] == 0, (tx, rx)
    assert "REGISTERED device-buffer owner 2 now-backed-by 5" in rx[1] + tx[1]     # (2 + 3) % 8
    assert "re-homed GPU 2 -> GPU 5" in rx[2] + tx[2]
    assert "DIRECT bytes 0 msgs 0" in tx[1]


def test_same_host_direct_path_writes_the_exported_receive_buffer():
    """With the side channel on (the default once device buffers are enabled) the receiver exports the cuMem
    allocation behind its registered buffer over a Unix socket, the sender maps it and stores every chunk straight
    into it: all payload bytes are counted as direct, none cross the TCP data sockets, and the receiver (which
    compares against the generator) still sees the right bytes -- in a buffer that was re-homed to the relay GPU."""
    env = {"FUSELINK_CUDA_PTRS": "1", "FUSELINK_VMM_FAKE": "1", "FUSELINK_VMM_FAKE_NGPUS": "8", "FL_HARNESS_VERBOSE": "1"}
    sizes = [3 << 20, 70000, 0, 5]
    tx, rx = _pair(sizes, env=env, common=["--device-buffers", "--dev", "2", "--chunk", "524288"],
                   extra_recv=["--channel", "3"], extra_send=[])
    assert tx[0] == 0 and rx[0] == 0, (tx, rx)
    total = sum(sizes)
    nmsgs = 6 + 1 + 0 + 1                                         # chunks with a payload; the empty message has nothing to store
    assert f"DIRECT bytes {total} msgs {nmsgs} of {total} bytes" in tx[1], tx[1]
    assert "re-homed GPU 2 -> GPU 5" in rx[2] + tx[2]
    assert "mapped at" in tx[2]
    # the harness registers a fresh buffer per message and deregisters it afterwards: the sender unmaps what the receiver
    # has let go of, so at most the last region is still mapped at the end (its notice may arrive after the last send)
    mapped = int([l for l in tx[1].splitlines() if l.startswith("PEER-REGIONS-MAPPED")][0].split()[1])
    assert mapped <= 1, tx[1]


def test_direct_path_is_negotiated_per_connection():
    """A sender that does not open the side channel (as one on another host cannot) gets the staged path from a
    receiver that offers it."""
    env = {"FUSELINK_CUDA_PTRS": "1", "FUSELINK_VMM_FAKE": "1", "FUSELINK_VMM_FAKE_NGPUS": "2"}
    tx, rx = _pair([1 << 20, 17], env=env, env_send={"FUSELINK_NVL": "0"}, common=["--device-buffers", "--chunk", "262144"])
    assert tx[0] == 0 and rx[0] == 0, (tx, rx)
    assert "DIRECT bytes 0 msgs 0" in tx[1]


def test_direct_path_over_several_channels():
    env = {"FUSELINK_CUDA_PTRS": "1", "FUSELINK_VMM_FAKE": "1", "FUSELINK_VMM_FAKE_NGPUS": "4", "FUSELINK_TCP_NDEV": "4"}
    tx, rx = _pair([(8 << 20) + 12], env=env, common=["--device-buffers", "--channels", "4", "--chunk", "1048576", "--inflight", "4"])
    assert tx[0] == 0 and rx[0] == 0, (tx, rx)
    assert f"DIRECT bytes {(8 << 20) + 12} " in tx[1], tx[1]


def test_device_buffers_refused_unless_enabled():
    tx, rx = _pair([4096], common=["--device-buffers"], env={"FUSELINK_VMM_FAKE": "1"}, timeout=30)
    assert tx[0] != 0 and rx[0] != 0


def test_plugin_symbols_and_properties():
    lib = ctypes.CDLL(PLUGIN)
    for sym in ("ncclNetPlugin_v6", "ncclNetPlugin_v7", "ncclNetPlugin_v8"):
        assert hasattr(lib, sym)
    name = ctypes.c_char_p.in_dll(lib, "ncclNetPlugin_v7")
    assert name.value == b"FuseLink"


def test_hca_filter_syntax():
    lib = ctypes.CDLL(PLUGIN)
    f = lib.fuselink_hca_allowed
    f.argtypes = [ctypes.c_char_p, ctypes.c_char_p, ctypes.c_int]
    assert f(b"", b"mlx5_0", 1) == 1
    assert f(b"mlx5", b"mlx5_3", 1) == 1                       # prefix match
    assert f(b"=mlx5_1", b"mlx5_10", 1) == 0                   # exact
    assert f(b"^mlx5_1", b"mlx5_1", 1) == 0 and f(b"^mlx5_1", b"mlx5_2", 1) == 1
    assert f(b"mlx5_0:2", b"mlx5_0", 1) == 0 and f(b"mlx5_0:2", b"mlx5_0", 2) == 1
    spec = b"=mlx5_0,3,4,5,6,9,10,11"                          # the reference's 8-NIC list
    allowed = [i for i in range(12) if f(spec, f"mlx5_{i}".encode(), 1)]
    assert allowed == [0, 3, 4, 5, 6, 9, 10, 11]


def test_refused_connect_is_retried_within_a_budget():
    """Nothing listens at the address of the handle: the sender retries the refused connection 1 ms apart and gives up
    after FUSELINK_CONNECT_RETRIES attempts with an error, instead of failing at the first refusal or spinning forever."""
    import socket
    import struct
    import time
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()                                                            # a port nobody listens on
    v4mapped = b"\x00" * 10 + b"\xff\xff" + socket.inet_aton("127.0.0.1")
    sockaddr_in6 = struct.pack("<H", socket.AF_INET6) + struct.pack(">H", port) + struct.pack("<I", 0) + v4mapped + struct.pack("<I", 0)
    handle = struct.pack("<Q", 0x464c4e4b48444c31) + sockaddr_in6 + struct.pack("<iiii", 0, 4, 0, 0)
    handle = handle.ljust(56, b"\x00") + struct.pack("<QQ", 0, 0)
    handle = handle.ljust(128, b"\x00")
    with tempfile.TemporaryDirectory() as d:
        hf = os.path.join(d, "handle")
        open(hf, "wb").write(handle)
        e = dict(os.environ, NCCL_SOCKET_IFNAME="lo", FUSELINK_CONNECT_RETRIES="150")
        t0 = time.time()
        tx = subprocess.run([HARNESS, PLUGIN, "send", hf, "4096"], env=e, capture_output=True, text=True, timeout=60)
        dt = time.time() - t0
    assert tx.returncode == 2 and "connect failed" in tx.stderr
    assert "after 150 retries" in tx.stderr, tx.stderr
    assert 0.15 <= dt < 30


def test_registering_a_sub_range_takes_over_the_whole_allocation():
    """NCCL registers buffers that start inside a larger cuMem allocation: the plugin finds the mapping the pointer lies
    in, re-homes that whole mapping (contents kept) and exports it; the direct path then writes at the right offset."""
    env = {"FUSELINK_CUDA_PTRS": "1", "FUSELINK_VMM_FAKE": "1", "FUSELINK_VMM_FAKE_NGPUS": "8", "FL_HARNESS_VERBOSE": "1"}
    sizes = [(1 << 20) + 40, 4096]
    tx, rx = _pair(sizes, env=env, common=["--device-buffers", "--dev", "1", "--reg-offset", str((2 << 20) + 256), "--chunk", "262144"],
                   extra_recv=["--channel", "2"])
    assert tx[0] == 0 and rx[0] == 0, (tx, rx)
    assert "re-homed GPU 1 -> GPU 3" in rx[2] + tx[2]
    assert f"DIRECT bytes {sum(sizes)} " in tx[1], tx[1]


@pytest.mark.parametrize("transport", ["tcp", "rdma-soft"])
def test_stray_and_malformed_connections_do_not_disturb_a_transfer(transport):
    """Port scanners and broken peers: random bytes, truncated hellos, hellos with a valid magic and nonsense fields,
    and connections that say nothing arrive at the listener before and while the real sender connects.  They are dropped
    (the reference validates magic and type the same way, src/extern/socket.cc:431-437) and the transfer is bit-exact."""
    import random
    import socket
    import struct
    import time
    extra = {} if transport == "tcp" else {"FUSELINK_TRANSPORT": "rdma", "FUSELINK_RDMA_PROVIDER": "soft"}
    rng = random.Random(7)
    with tempfile.TemporaryDirectory() as d:
        hf = os.path.join(d, "handle")
        e = dict(os.environ, NCCL_SOCKET_IFNAME="lo", NCCL_SOCKET_FAMILY="AF_INET", **extra)
        sizes = [str(1 << 20), "4097"]
        rx = subprocess.Popen([HARNESS, PLUGIN, "recv", hf, "--chunk", "131072", *sizes], env=e, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
        keep = []
        try:
            t0 = time.time()
            while not os.path.exists(hf):
                assert time.time() - t0 < 20
                time.sleep(0.01)
            port = struct.unpack("!H", open(hf, "rb").read()[10:12])[0]
            magic = 0x464c4e4b48454c4f

            def junk(i):
                kind = i % 6
                if kind == 0:
                    return bytes(rng.randrange(256) for _ in range(rng.randrange(1, 200)))
                if kind == 1:
                    return struct.pack("<QQ", magic, 1)                                        # truncated hello
                if kind == 2:
                    return struct.pack("<QQiiii", magic, rng.getrandbits(60), 1, 99, 0, 4)     # data socket of device 99
                if kind == 3:
                    return struct.pack("<QQiiii", magic, rng.getrandbits(60), 0, -1, 0, 4000)  # absurd device count
                if kind == 4:
                    return struct.pack("<QQiiii", magic ^ 1, 5, 0, -1, 0, 4)                   # wrong magic
                return b""                                                                     # connects and says nothing

            for i in range(24):
                s = socket.create_connection(("127.0.0.1", port))
                b = junk(i)
                if b:
                    s.sendall(b)
                if i % 3 == 0:
                    keep.append(s)                        # some stay open for the whole transfer
                else:
                    s.close()
            tx = subprocess.run([HARNESS, PLUGIN, "send", hf, "--chunk", "131072", *sizes], env=e, capture_output=True, text=True, timeout=90)
            out, err = rx.communicate(timeout=60)
        finally:
            for s in keep:
                s.close()
            if rx.poll() is None:
                rx.kill()
        assert tx.returncode == 0, (tx.stdout, tx.stderr)
        assert rx.returncode == 0 and "OK received" in out, (out, err)


def _xfer_gbs(out):
    line = [l for l in out.splitlines() if l.startswith("OK ")][0]
    return float(line.split("(")[2].split()[0])


def test_striping_over_rate_limited_nics_adds_their_bandwidth():
    """The reference's central claim in miniature: one transfer held to the line rate of its own NIC gets the sum of the
    rates of the idle NICs it is striped over.  Eight virtual NICs of 200 MB/s each; degree 1, 2 and 4."""
    got = {}
    for degree in (1, 2, 4):
        env = {"FUSELINK_TCP_NDEV": "8", "FUSELINK_TCP_NIC_MBPS": "200", "NCCL_FUSELINK_DEGREE": str(degree), "NCCL_FUSELINK_STEP": "1",
               "FUSELINK_MIN_STRIPE_BYTES": "65536"}
        tx, rx = _pair([96 << 20], env=env, common=["--chunk", "1048576", "--inflight", "8"], timeout=120)
        assert tx[0] == 0 and rx[0] == 0, (tx, rx)
        got[degree] = _xfer_gbs(rx[1])
    assert 0.15 < got[1] < 0.26, got                       # one NIC: its 0.2 GB/s
    assert got[2] > 1.6 * got[1] and got[4] > 3.0 * got[1], got


def _two_jobs(env, size=48 << 20):
    """Two sender/receiver pairs at the same time (four processes); returns the transfer rate each receiver saw."""
    procs, dirs = [], []
    try:
        for j in range(2):
            d = tempfile.mkdtemp()
            dirs.append(d)
            hf = os.path.join(d, "handle")
            e = dict(os.environ, NCCL_SOCKET_IFNAME="lo", **env)
            args = ["--chunk", "1048576", "--inflight", "8", str(size)]
            rx = subprocess.Popen([HARNESS, PLUGIN, "recv", hf, *args], env=e, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
            tx = subprocess.Popen([HARNESS, PLUGIN, "send", hf, *args], env=e, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
            procs.append((tx, rx))
        rates = []
        for tx, rx in procs:
            txo, txe = tx.communicate(timeout=180)
            rxo, rxe = rx.communicate(timeout=180)
            assert tx.returncode == 0 and rx.returncode == 0, (txo, txe, rxo, rxe)
            rates.append(_xfer_gbs(rxo))
        return rates
    finally:
        import shutil
        for tx, rx in procs:
            for p in (tx, rx):
                if p.poll() is None:
                    p.kill()
        for d in dirs:
            shutil.rmtree(d, ignore_errors=True)


def test_two_jobs_contend_for_one_nic_unless_the_monitor_is_shared():
    """The contention scenario of the reference's two-task experiment (experiments/serving/run_test_twotask.sh): two jobs
    whose traffic would land on the same NIC.  The NICs are shared between the processes (line-rate buckets in shared
    memory, 200 MB/s each).  Without the monitor both jobs sit on NIC 0 and split it; with one monitor table shared by
    all four processes each job takes an idle NIC and runs at line rate."""
    import uuid
    tag = uuid.uuid4().hex[:10]
    nic_shm, mon_shm = f"/fl_nic_{tag}", f"/fl_mon_{tag}"
    base = {"FUSELINK_TCP_NDEV": "8", "FUSELINK_TCP_NIC_MBPS": "200", "FUSELINK_TCP_NIC_SHM": nic_shm, "NCCL_FUSELINK_DEGREE": "1"}
    daemon = None
    try:
        alone = _two_jobs(dict(base, FUSELINK_MONITOR="0"))
        exe = os.path.join(os.path.dirname(HARNESS), "fuselink-monitor")
        daemon = subprocess.Popen([exe, "--shm", mon_shm, "--groups", "8", "--seconds", "120"], stdout=subprocess.PIPE, text=True)
        daemon.stdout.readline()                                   # table is up
        shared = _two_jobs(dict(base, FUSELINK_MONITOR_SHM=mon_shm))
        striped = _two_jobs(dict(base, FUSELINK_MONITOR_SHM=mon_shm, NCCL_FUSELINK_DEGREE="2", FUSELINK_MIN_STRIPE_BYTES="65536"))
    finally:
        if daemon is not None:
            daemon.terminate()
            daemon.wait(timeout=10)
        for n in (nic_shm, mon_shm):
            try:
                os.unlink("/dev/shm" + n)
            except OSError:
                pass
    assert sum(alone) < 0.26 and max(alone) < 0.19, alone         # one 0.2 GB/s NIC for both
    assert min(shared) > 0.16, shared                              # a NIC each
    assert sum(shared) > 1.5 * sum(alone), (alone, shared)
    # degree 2: the second stripe of each job goes to a NIC the shared table shows idle, not blindly to the neighbour's
    assert min(striped) > 0.3, striped


def test_makefile_builds_a_working_plugin_without_python(tmp_path):
    """`make fl monitor harness` (the reference's target names, Makefile:33-49) into a scratch directory: the plugin it links
    moves data between two processes and the monitor daemon starts."""
    import shutil
    if not shutil.which("make") or not shutil.which(os.environ.get("CXX", "g++")):
        pytest.skip("no make / C++ compiler")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = str(tmp_path / "b")
    b = subprocess.run(["make", "-C", root, "-j8", f"BUILD={out}", "OPT=-O1", "fl", "monitor", "harness"], capture_output=True, text=True, timeout=900)
    assert b.returncode == 0, b.stdout[-2000:] + b.stderr[-3000:]
    harness, plugin = os.path.join(out, "bin", "fl_net_harness"), os.path.join(out, "lib", "libnccl-net-fuselink.so")
    hf = str(tmp_path / "h")
    env = dict(os.environ, NCCL_SOCKET_IFNAME="lo", NCCL_FUSELINK_DEGREE="2", FUSELINK_MIN_STRIPE_BYTES="65536")
    rx = subprocess.Popen([harness, plugin, "recv", hf, "--chunk", "262144", str(3 << 20), "77"], env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
    tx = subprocess.Popen([harness, plugin, "send", hf, "--chunk", "262144", str(3 << 20), "77"], env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
    txo, txe = tx.communicate(timeout=120)
    rxo, rxe = rx.communicate(timeout=120)
    assert tx.returncode == 0 and rx.returncode == 0 and "OK received" in rxo, (txo, txe, rxo, rxe)
    mon = subprocess.run([os.path.join(out, "bin", "fuselink-monitor"), "--shm", f"/fl_mk_{os.getpid()}", "--groups", "4", "--seconds", "0.2"],
                         capture_output=True, text=True, timeout=30)
    assert mon.returncode == 0, mon.stdout + mon.stderr
