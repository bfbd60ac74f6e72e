"""The RDMA transport of the plugin (receiver-written descriptor FIFO, RDMA write + write-with-immediate, striping
over devices and queue pairs) driven through the ncclNet entry points by two processes, on the software NIC that
stands in for libibverbs devices.  Same harness and the same bitwise checks as the TCP transport."""
import os

import pytest

from test_plugin_cpu import PLUGIN, _pair

SOFT = {"FUSELINK_TRANSPORT": "rdma", "FUSELINK_RDMA_PROVIDER": "soft", "FUSELINK_SOFT_NDEV": "4"}


def _counters(out):
    line = [l for l in out.splitlines() if l.startswith("RDMA messages")]
    assert line, out
    w = line[0].split()
    return int(w[2]), int(w[4]), int(w[6])


@pytest.mark.parametrize("abi", [6, 7, 8])
def test_bitwise_transfer_reference_config(abi):
    tx, rx = _pair([4096, 1 << 20, 64 << 20], env=SOFT, common=["--abi", str(abi), "--chunk", "524288", "--inflight", "8"])
    assert tx[0] == 0 and rx[0] == 0, (tx, rx)
    msgs, pieces, wrs = _counters(tx[1])
    assert msgs == 1 + 2 + 128 and pieces == msgs                    # degree 1: one piece per chunk
    # the software NIC is an Ethernet (RoCE-like) device: adaptive routing is off by default, so every message is its
    # 16-byte size record plus one write-with-immediate that carries the payload
    assert wrs == 131 * 2


def test_adaptive_routing_splits_large_writes():
    """NCCL_IB_ADAPTIVE_ROUTING=1: above NCCL_IB_AR_THRESHOLD the payload goes as a plain write followed by an empty
    write-with-immediate; at or below it one write-with-immediate carries everything."""
    env = dict(SOFT, NCCL_IB_ADAPTIVE_ROUTING="1")
    tx, rx = _pair([4096, 1 << 20], env=env, common=["--chunk", "524288", "--inflight", "8"])
    assert tx[0] == 0 and rx[0] == 0, (tx, rx)
    msgs, pieces, wrs = _counters(tx[1])
    assert msgs == 3 and wrs == 2 + 2 * 3
    env = dict(SOFT, NCCL_IB_ADAPTIVE_ROUTING="1", NCCL_IB_AR_THRESHOLD=str(1 << 20))
    tx, rx = _pair([4096, 1 << 20], env=env, common=["--chunk", "524288", "--inflight", "8"])
    assert tx[0] == 0 and rx[0] == 0, (tx, rx)
    assert _counters(tx[1])[2] == 3 * 2


def test_odd_sizes_zero_length_and_many_in_flight():
    tx, rx = _pair([0, 1, 3, 4097, 8192, 8193, 524289, 1234567], env=SOFT, common=["--chunk", "4096", "--inflight", "64"])
    assert tx[0] == 0 and rx[0] == 0, (tx, rx)


def test_striping_over_devices_and_queue_pairs():
    """NCCL_FUSELINK_DEGREE devices x NCCL_IB_QPS_PER_CONNECTION queue pairs: every 1 MiB chunk becomes 2 x 2 pieces
    in multiples of 128 bytes."""
    env = dict(SOFT, NCCL_FUSELINK_DEGREE="2", NCCL_FUSELINK_STEP="1", FUSELINK_MIN_STRIPE_BYTES="65536",
               NCCL_IB_QPS_PER_CONNECTION="2", NCCL_IB_SPLIT_DATA_ON_QPS="1")
    tx, rx = _pair([8 << 20, (1 << 20) + 77], env=env, common=["--chunk", "1048576", "--inflight", "8"])
    assert tx[0] == 0 and rx[0] == 0, (tx, rx)
    msgs, pieces, _ = _counters(tx[1])
    assert msgs == 8 + 2
    assert pieces == 9 * 4 + 1                                       # the 77-byte tail is too small to cut


def test_round_robin_over_queue_pairs_without_splitting():
    env = dict(SOFT, NCCL_IB_QPS_PER_CONNECTION="4", NCCL_IB_SPLIT_DATA_ON_QPS="0", NCCL_IB_USE_INLINE="1")
    tx, rx = _pair([4 << 20], env=env, common=["--chunk", "262144", "--inflight", "16"])
    assert tx[0] == 0 and rx[0] == 0, (tx, rx)
    msgs, pieces, _ = _counters(tx[1])
    assert msgs == pieces == 16


def test_four_channels_with_the_monitor_choosing_devices():
    env = dict(SOFT, FUSELINK_SOFT_NDEV="8", NCCL_FUSELINK_DEGREE="2", FUSELINK_MIN_STRIPE_BYTES="65536")
    tx, rx = _pair([32 << 20, 3], env=env, common=["--channels", "4", "--chunk", "524288", "--inflight", "8"])
    assert tx[0] == 0 and rx[0] == 0, (tx, rx)
    assert "channels 4" in rx[1]


def test_one_thread_per_channel():
    env = dict(SOFT, NCCL_FUSELINK_DEGREE="2", FUSELINK_MIN_STRIPE_BYTES="65536", NCCL_IB_QPS_PER_CONNECTION="2")
    tx, rx = _pair([8 << 20, 4097, 0], env=env, common=["--channels", "4", "--threads", "--chunk", "262144", "--inflight", "8"])
    assert tx[0] == 0 and rx[0] == 0, (tx, rx)
    assert f"OK received {4 * ((8 << 20) + 4097)} bytes" in rx[1]


def test_wrong_remote_key_is_refused_by_the_responder():
    """The responder checks key and bounds of every write; a bad key comes back as a remote-access completion error,
    the queue pair goes to the error state and the connection reports it instead of corrupting memory."""
    env = dict(SOFT, FUSELINK_FAULT_BAD_RKEY_AFTER="3", FUSELINK_NET_TIMEOUT_MS="2000")
    tx, rx = _pair([1 << 20], env=env, common=["--chunk", "65536", "--expect-error"], timeout=60)
    assert tx[0] == 0 and "EXPECTED-ERROR" in tx[1], tx
    assert rx[0] == 0 and "EXPECTED-ERROR" in rx[1], rx            # the receiver's request never completes: timeout
    assert "status 10" in tx[2]


def test_sender_death_is_detected_by_the_receiver():
    env = dict(SOFT, FUSELINK_NET_TIMEOUT_MS="1500")
    tx, rx = _pair([8 << 20], env=env, common=["--chunk", "524288"], extra_send=["--die-after-chunks", "3"],
                   extra_recv=["--expect-error"], timeout=60)
    assert tx[0] == 9
    assert rx[0] == 0 and "EXPECTED-ERROR" in rx[1], rx


def test_device_buffers_travel_by_rdma_after_rehoming():
    env = dict(SOFT, FUSELINK_CUDA_PTRS="1", FUSELINK_VMM_FAKE="1", FUSELINK_VMM_FAKE_NGPUS="8", FL_HARNESS_VERBOSE="1")
    tx, rx = _pair([3 << 20, 70000], env=env, common=["--device-buffers", "--dev", "2", "--chunk", "524288"], extra_recv=["--channel", "3"])
    assert tx[0] == 0 and rx[0] == 0, (tx, rx)
    assert "re-homed GPU 2 -> GPU 5" in rx[2] + tx[2]


def test_asynchronous_device_event_is_logged():
    env = dict(SOFT, FL_HARNESS_VERBOSE="1")
    tx, rx = _pair([4096], env=env, extra_recv=["--inject-event", "port error (injected)"])
    assert tx[0] == 0 and rx[0] == 0, (tx, rx)
    assert "asynchronous event: port error (injected)" in rx[2]


def test_properties_come_from_the_provider():
    """With the RDMA transport the devices NCCL sees are the provider's ports."""
    import subprocess, sys, textwrap
    code = textwrap.dedent(f"""
        import ctypes
        lib = ctypes.CDLL({PLUGIN!r})
        class V7(ctypes.Structure):
            _fields_ = [("name", ctypes.c_char_p), ("init", ctypes.CFUNCTYPE(ctypes.c_int, ctypes.c_void_p)),
                        ("devices", ctypes.CFUNCTYPE(ctypes.c_int, ctypes.POINTER(ctypes.c_int))),
                        ("props", ctypes.CFUNCTYPE(ctypes.c_int, ctypes.c_int, ctypes.c_void_p))]
        v7 = V7.in_dll(lib, "ncclNetPlugin_v7")
        assert v7.init(None) == 0
        n = ctypes.c_int(0); v7.devices(ctypes.byref(n))
        buf = ctypes.create_string_buffer(256)
        assert v7.props(1, buf) == 0
        name = ctypes.cast(buf, ctypes.POINTER(ctypes.c_char_p))[0]
        print(n.value, name.decode())
    """)
    out = subprocess.run([sys.executable, "-c", code], env=dict(os.environ, **SOFT), capture_output=True, text=True, timeout=60)
    assert out.returncode == 0, out.stderr
    assert out.stdout.split() == ["4", "softnic_1"]


def test_flush_reads_device_memory_back_through_the_nic():
    """NCCL_GDR_FLUSH_DISABLE=0: iflush on a device buffer posts a one-byte RDMA read on a queue pair connected to itself
    and completes through test(); with the default (disabled, as the reference sets it) iflush returns no request."""
    base = dict(SOFT, FUSELINK_CUDA_PTRS="1", FUSELINK_VMM_FAKE="1", FUSELINK_VMM_FAKE_NGPUS="2")
    tx, rx = _pair([1 << 20, 4097], env=dict(base, NCCL_GDR_FLUSH_DISABLE="0"), common=["--device-buffers", "--chunk", "262144"], extra_recv=["--flush"])
    assert tx[0] == 0 and rx[0] == 0, (tx, rx)
    assert "FLUSHES 2" in rx[1]
    tx, rx = _pair([1 << 20], env=base, common=["--device-buffers", "--chunk", "262144"], extra_recv=["--flush"])
    assert tx[0] == 0 and rx[0] == 0, (tx, rx)
    assert "FLUSHES 0" in rx[1]


def test_device_failure_on_the_sender_moves_pieces_to_another_device():
    """One device's link dies in the middle of a message (the software NIC breaks its queue pair after 3 MB): the
    completion error marks the device dead for the connection, the affected pieces are posted again on the next device,
    the receiver counts each piece once, and every byte arrives."""
    env = dict(SOFT, NCCL_FUSELINK_DEGREE="2", FUSELINK_MIN_STRIPE_BYTES="65536", FL_HARNESS_VERBOSE="1", FUSELINK_NET_TIMEOUT_MS="8000")
    tx, rx = _pair([16 << 20, 1 << 20, 7], env=env, common=["--chunk", "524288", "--inflight", "8"], timeout=90,
                   env_send={"FUSELINK_SOFT_FAULT_DEV": "0", "FUSELINK_SOFT_FAULT_AFTER_BYTES": str(3 << 20)})
    assert tx[0] == 0 and rx[0] == 0, (tx, rx)
    assert "RDMA-FAILOVERS" in tx[1] and "is given up; traffic moves to device" in tx[2], tx


def test_device_failure_under_the_descriptor_writes_is_survived():
    """The device that carries the receiver's descriptor writes dies: the receiver moves them to another device and
    writes the descriptors of its unfinished receives again."""
    env = dict(SOFT, FL_HARNESS_VERBOSE="1", FUSELINK_NET_TIMEOUT_MS="8000")
    tx, rx = _pair([8 << 20, 3], env=env, common=["--chunk", "262144", "--inflight", "8"], timeout=90,
                   env_recv={"FUSELINK_SOFT_FAULT_DEV": "0", "FUSELINK_SOFT_FAULT_AFTER_BYTES": "1500"})
    assert tx[0] == 0 and rx[0] == 0, (tx, rx)
    assert "RDMA-FAILOVERS" in rx[1] and "is given up" in rx[2], rx


def test_failover_can_be_switched_off():
    env = dict(SOFT, NCCL_FUSELINK_DEGREE="2", FUSELINK_MIN_STRIPE_BYTES="65536", FUSELINK_FAILOVER="0", FUSELINK_NET_TIMEOUT_MS="2000")
    tx, rx = _pair([16 << 20], env=env, common=["--chunk", "524288", "--expect-error"], timeout=60,
                   env_send={"FUSELINK_SOFT_FAULT_DEV": "0", "FUSELINK_SOFT_FAULT_AFTER_BYTES": str(3 << 20)})
    assert tx[0] == 0 and "EXPECTED-ERROR" in tx[1], tx


def test_striping_over_rate_limited_devices_adds_their_bandwidth():
    """Same experiment as on the TCP transport: eight software devices of 200 MB/s, one connection, degree 1 / 2 / 4."""
    from test_plugin_cpu import _xfer_gbs
    got = {}
    for degree in (1, 2, 4):
        env = dict(SOFT, FUSELINK_SOFT_NDEV="8", FUSELINK_TCP_NIC_MBPS="200", NCCL_FUSELINK_DEGREE=str(degree), FUSELINK_MIN_STRIPE_BYTES="65536")
        tx, rx = _pair([64 << 20], env=env, common=["--chunk", "1048576", "--inflight", "8"], timeout=120)
        assert tx[0] == 0 and rx[0] == 0, (tx, rx)
        got[degree] = _xfer_gbs(rx[1])
    assert 0.15 < got[1] < 0.26, got
    assert got[2] > 1.6 * got[1] and got[4] > 3.0 * got[1], got


def _build_fake_ibverbs(tmp_path):
    """tests/fake_ibverbs/fake_ibverbs.cc + the software NIC as `libibverbs.so.1` in a directory of its own."""
    import shutil
    import subprocess
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    net = os.path.join(root, "fuselink_b200", "csrc", "net")
    cxx = next((c for c in (os.environ.get("CXX"), "g++", "/usr/bin/g++") if c and shutil.which(c)), None)
    if cxx is None:
        pytest.skip("no C++ compiler")
    out = os.path.join(str(tmp_path), "libibverbs.so.1")
    srcs = [os.path.join(root, "tests", "fake_ibverbs", "fake_ibverbs.cc")] + [os.path.join(net, f) for f in
                                                                              ("soft_provider.cc", "nic_rate.cc", "params.cc", "logging.cc")]
    b = subprocess.run([cxx, "-O1", "-g", "-std=c++17", "-fPIC", "-shared", "-pthread", "-o", out, *srcs, "-lrt"], capture_output=True, text=True, timeout=600)
    assert b.returncode == 0, b.stderr[-3000:]
    return str(tmp_path)


def test_verbs_provider_end_to_end_against_a_fake_libibverbs(tmp_path):
    """The libibverbs provider (dlopen, device / port discovery, NCCL_IB_HCA, queue pairs through INIT -> RTR -> RTS with the
    attribute masks the library insists on, work-request and completion translation through the function table inside the
    context) carrying real transfers: the library it loads is a stand-in with the real calling conventions."""
    libdir = _build_fake_ibverbs(tmp_path)
    env = {"FUSELINK_TRANSPORT": "rdma", "LD_LIBRARY_PATH": libdir + ":" + os.environ.get("LD_LIBRARY_PATH", ""), "FUSELINK_FAKE_IB_NDEV": "3",
           "FUSELINK_SOFT_NDEV": "4", "NCCL_FUSELINK_DEGREE": "2", "FUSELINK_MIN_STRIPE_BYTES": "65536", "NCCL_IB_QPS_PER_CONNECTION": "2",
           "FL_HARNESS_VERBOSE": "1"}
    tx, rx = _pair([4096, 3 << 20, 0, 70001], env=env, common=["--chunk", "524288", "--inflight", "8"])
    assert tx[0] == 0 and rx[0] == 0, (tx, rx)
    assert "3 device(s) through the verbs provider" in tx[2] and "3 device(s) over RDMA" in tx[2], tx[2]
    msgs, pieces, _ = _counters(tx[1])
    assert msgs == 1 + 6 + 1 + 1 and pieces > msgs                   # stripes over two devices x two queue pairs
    # the HCA filter picks devices by name, exactly
    tx, rx = _pair([1 << 20], env=dict(env, NCCL_IB_HCA="=mlx5_1,2"), common=["--chunk", "262144"])
    assert tx[0] == 0 and rx[0] == 0, (tx, rx)
    assert "2 device(s) through the verbs provider" in tx[2]
    # NCCL_IB_DISABLE=1 turns the provider off: the plugin falls back to TCP
    tx, rx = _pair([1 << 20], env=dict(env, NCCL_IB_DISABLE="1", FUSELINK_TRANSPORT="auto"), common=["--chunk", "262144"])
    assert tx[0] == 0 and rx[0] == 0 and "over TCP" in tx[2], (tx, rx)


def test_properties_of_a_verbs_device(tmp_path):
    """Speed from the width and rate codes (4x EDR = 100 Gb/s), the port that is down is skipped, maxComms = max_qp."""
    import subprocess, sys, textwrap
    libdir = _build_fake_ibverbs(tmp_path)
    code = textwrap.dedent(f"""
        import ctypes
        lib = ctypes.CDLL({PLUGIN!r})
        class Props(ctypes.Structure):
            _fields_ = [("name", ctypes.c_char_p), ("pci", ctypes.c_char_p), ("guid", ctypes.c_uint64), ("ptr", ctypes.c_int), ("speed", ctypes.c_int),
                        ("port", ctypes.c_int), ("latency", ctypes.c_float), ("maxComms", ctypes.c_int), ("maxRecvs", ctypes.c_int)]
        class V6(ctypes.Structure):
            _fields_ = [("name", ctypes.c_char_p), ("init", ctypes.CFUNCTYPE(ctypes.c_int, ctypes.c_void_p)),
                        ("devices", ctypes.CFUNCTYPE(ctypes.c_int, ctypes.POINTER(ctypes.c_int))),
                        ("props", ctypes.CFUNCTYPE(ctypes.c_int, ctypes.c_int, ctypes.POINTER(Props)))]
        v6 = V6.in_dll(lib, "ncclNetPlugin_v6")
        assert v6.init(None) == 0
        n = ctypes.c_int(0); v6.devices(ctypes.byref(n))
        p = Props(); assert v6.props(1, ctypes.byref(p)) == 0
        print(n.value, p.name.decode(), p.speed, p.maxComms, p.maxRecvs, hex(p.guid))
    """)
    env = dict(os.environ, FUSELINK_TRANSPORT="rdma", LD_LIBRARY_PATH=libdir + ":" + os.environ.get("LD_LIBRARY_PATH", ""), FUSELINK_FAKE_IB_NDEV="2")
    out = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=60)
    assert out.returncode == 0, out.stderr
    assert out.stdout.split() == ["2", "mlx5_1", "100000", "4096", "1", "0xfa4e000000000001"]


def test_verbs_provider_error_completions_and_reads(tmp_path):
    """Through the stand-in library too: a queue pair that breaks reports "retry exceeded" and its pieces move to another
    device; the flush is an RDMA READ work request on a queue pair connected to itself."""
    libdir = _build_fake_ibverbs(tmp_path)
    env = {"FUSELINK_TRANSPORT": "rdma", "LD_LIBRARY_PATH": libdir + ":" + os.environ.get("LD_LIBRARY_PATH", ""), "FUSELINK_FAKE_IB_NDEV": "4",
           "NCCL_FUSELINK_DEGREE": "2", "FUSELINK_MIN_STRIPE_BYTES": "65536", "FL_HARNESS_VERBOSE": "1", "FUSELINK_NET_TIMEOUT_MS": "8000"}
    tx, rx = _pair([8 << 20, 9], env=env, common=["--chunk", "524288", "--inflight", "8"], timeout=90,
                   env_send={"FUSELINK_SOFT_FAULT_DEV": "0", "FUSELINK_SOFT_FAULT_AFTER_BYTES": str(2 << 20)})
    assert tx[0] == 0 and rx[0] == 0, (tx, rx)
    assert "RDMA-FAILOVERS" in tx[1] and "completion status 12" in tx[2], tx
    flush = dict(env, FUSELINK_CUDA_PTRS="1", FUSELINK_VMM_FAKE="1", FUSELINK_VMM_FAKE_NGPUS="2", NCCL_GDR_FLUSH_DISABLE="0")
    tx, rx = _pair([1 << 20], env=flush, common=["--device-buffers", "--chunk", "262144"], extra_recv=["--flush"])
    assert tx[0] == 0 and rx[0] == 0, (tx, rx)
    assert "FLUSHES 1" in rx[1]


def test_phase_timers_are_printed_at_close():
    """FUSELINK_TIMERS=1: the run-time version of the timers the reference compiles out (isend, irecv, descriptor post,
    completion polling)."""
    tx, rx = _pair([1 << 20], env=dict(SOFT, FUSELINK_TIMERS="1"), common=["--chunk", "262144"])
    assert tx[0] == 0 and rx[0] == 0, (tx, rx)
    assert "[fuselink timer] rdma send isend" in tx[2] and "[fuselink timer] rdma send progress" in tx[2]
    assert "[fuselink timer] rdma recv irecv" in rx[2] and "[fuselink timer] rdma recv post_desc" in rx[2]


def test_verbs_attributes_follow_the_environment(tmp_path):
    """NCCL_IB_GID_INDEX / _TIMEOUT / _RETRY_CNT / _PKEY / _SL / _TC / _USE_INLINE / _PCI_RELAXED_ORDERING reach the calls of
    the verbs library with the values given (the stand-in library writes down what it is called with), and an asynchronous
    port event is fetched, logged and acknowledged by the watcher thread."""
    libdir = _build_fake_ibverbs(tmp_path)
    log = os.path.join(str(tmp_path), "calls.log")
    env = {"FUSELINK_TRANSPORT": "rdma", "LD_LIBRARY_PATH": libdir + ":" + os.environ.get("LD_LIBRARY_PATH", ""), "FUSELINK_FAKE_IB_NDEV": "2",
           "FUSELINK_FAKE_IB_LOG": log, "FUSELINK_FAKE_IB_EVENT_MS": "1", "FL_HARNESS_VERBOSE": "1",
           "NCCL_IB_GID_INDEX": "3", "NCCL_IB_TIMEOUT": "20", "NCCL_IB_RETRY_CNT": "5", "NCCL_IB_PKEY": "2", "NCCL_IB_SL": "4", "NCCL_IB_TC": "106",
           "NCCL_IB_USE_INLINE": "1", "NCCL_IB_PCI_RELAXED_ORDERING": "0"}
    tx, rx = _pair([1 << 20, 77], env=env, common=["--chunk", "262144"])
    assert tx[0] == 0 and rx[0] == 0, (tx, rx)
    calls = open(log).read().splitlines()
    kv = lambda l: dict(f.split("=") for f in l.split()[1:])
    init = [kv(l) for l in calls if l.startswith("init ")]
    rtr = [kv(l) for l in calls if l.startswith("rtr ")]
    rts = [kv(l) for l in calls if l.startswith("rts ")]
    qps = [kv(l) for l in calls if l.startswith("create_qp ")]
    mrs = [kv(l) for l in calls if l.startswith("reg_mr ")]
    assert init and len(init) == len(rtr) == len(rts)
    assert all(c["pkey"] == "2" and int(c["access"], 16) == 0x7 for c in init)
    assert all(c["sgid_index"] == "3" and c["tc"] == "106" and c["sl"] == "4" and c["hop_limit"] == "255" for c in rtr)
    assert all(c["timeout"] == "20" and c["retry_cnt"] == "5" and c["rnr_retry"] == "7" for c in rts)
    assert all(int(c["max_inline"]) >= 128 for c in qps if int(c["max_send_wr"]) > 1) and qps
    assert mrs and all(int(c["access"], 16) & (1 << 20) == 0 for c in mrs)           # relaxed ordering switched off
    assert any(l.startswith("ack_async_event type=10") for l in calls)
    assert "asynchronous event: port error" in tx[2] + rx[2]
    # relaxed ordering on: the flag is in every registration
    os.remove(log)
    tx, rx = _pair([1 << 20], env=dict(env, NCCL_IB_PCI_RELAXED_ORDERING="1", NCCL_IB_USE_INLINE="0"), common=["--chunk", "262144"])
    assert tx[0] == 0 and rx[0] == 0, (tx, rx)
    calls = open(log).read().splitlines()
    mrs = [kv(l) for l in calls if l.startswith("reg_mr ")]
    assert mrs and all(int(c["access"], 16) & (1 << 20) for c in mrs)
    assert all(c["max_inline"] == "0" for c in (kv(l) for l in calls if l.startswith("create_qp ")))


def _mr_counters(out):
    line = [l for l in out.splitlines() if l.startswith("MR registrations")]
    assert line, out
    w = line[0].split()
    return int(w[2]), int(w[4]), int(w[6])


def test_registration_cache_shares_a_buffer_between_channels():
    """NCCL registers one buffer once per connection: the second to fourth registration of the same pages is answered from
    the per-device cache (the reference's MR cache, src/plugin.cc:1265-1305)."""
    tx, rx = _pair([1 << 20], env=SOFT, common=["--chunk", "65536", "--channels", "4"])
    assert tx[0] == 0 and rx[0] == 0, (tx, rx)
    regs, hits, dmabuf = _mr_counters(tx[1])
    assert dmabuf == 0
    assert hits >= 3 * 4                                          # 3 repeated registrations x 4 devices
    one, _ = _pair([1 << 20], env=SOFT, common=["--chunk", "65536"])
    assert one[0] == 0
    regs1, hits1, _ = _mr_counters(one[1])
    assert regs - regs1 == 3 * 2 * 4 and hits1 == 0               # the extra connections add only their own FIFO + record registrations


def test_device_memory_is_registered_through_a_dmabuf_without_peer_memory():
    """No peer-memory module (FUSELINK_SOFT_PEERMEM=0): a device buffer reaches the NIC through a dma-buf descriptor the
    cuMem layer exports AFTER the buffer was re-homed, and the software NIC goes through its own mapping of that
    descriptor, never through the application's address."""
    env = dict(SOFT, FUSELINK_CUDA_PTRS="1", FUSELINK_VMM_FAKE="1", FUSELINK_VMM_FAKE_NGPUS="8", FL_HARNESS_VERBOSE="1", FUSELINK_SOFT_PEERMEM="0")
    tx, rx = _pair([3 << 20, 70000, 5], env=env, common=["--device-buffers", "--dev", "2", "--chunk", "524288", "--reg-offset", "4096"],
                   extra_recv=["--channel", "3"])
    assert tx[0] == 0 and rx[0] == 0, (tx, rx)
    assert "re-homed GPU 2 -> GPU 5" in rx[2]
    assert _mr_counters(tx[1])[2] == 3 * 4 and _mr_counters(rx[1])[2] == 3 * 4     # 3 buffers x 4 devices, both ends
    # with a peer-memory module the same buffers are registered by address
    tx, rx = _pair([3 << 20], env=dict(env, FUSELINK_SOFT_PEERMEM="1"), common=["--device-buffers", "--chunk", "524288"])
    assert tx[0] == 0 and rx[0] == 0 and _mr_counters(tx[1])[2] == 0, (tx, rx)


@pytest.mark.parametrize("remap", ["0", "1"])
def test_regmr_dmabuf_entry_point(remap):
    """regMrDmaBuf with a descriptor taken before the registration, as NCCL does.  A buffer the plugin leaves alone is
    registered through NCCL's descriptor; one it takes over (and re-homes) gets a fresh descriptor, because the old one
    names the memory the buffer no longer lives in."""
    env = dict(SOFT, FUSELINK_CUDA_PTRS="1", FUSELINK_VMM_FAKE="1", FUSELINK_VMM_FAKE_NGPUS="4", FL_HARNESS_VERBOSE="1", FUSELINK_SOFT_PEERMEM="0",
               FUSELINK_REMAP=remap, FUSELINK_NVL=remap)
    tx, rx = _pair([2 << 20, 4097], env=env, common=["--nccl-dmabuf", "--dev", "1", "--chunk", "262144"], extra_recv=["--channel", "2"])
    assert tx[0] == 0 and rx[0] == 0, (tx, rx)
    assert _mr_counters(rx[1])[2] == 2 * 4
    assert ("re-homed GPU 1 -> GPU 3" in rx[2]) == (remap == "1")


def test_pointer_support_follows_what_the_nics_can_reach():
    import subprocess, sys, textwrap
    code = textwrap.dedent(f"""
        import ctypes
        lib = ctypes.CDLL({PLUGIN!r})
        class Props(ctypes.Structure):
            _fields_ = [("name", ctypes.c_char_p), ("pci", ctypes.c_char_p), ("guid", ctypes.c_uint64), ("ptr", ctypes.c_int)]
        class V6(ctypes.Structure):
            _fields_ = [("name", ctypes.c_char_p), ("init", ctypes.CFUNCTYPE(ctypes.c_int, ctypes.c_void_p)),
                        ("devices", ctypes.CFUNCTYPE(ctypes.c_int, ctypes.POINTER(ctypes.c_int))),
                        ("props", ctypes.CFUNCTYPE(ctypes.c_int, ctypes.c_int, ctypes.c_void_p))]
        v6 = V6.in_dll(lib, "ncclNetPlugin_v6")
        assert v6.init(None) == 0
        buf = ctypes.create_string_buffer(256)
        assert v6.props(0, buf) == 0
        print(Props.from_buffer(buf).ptr)
    """)
    def ptr(**kw):
        env = {**os.environ, **SOFT, "FUSELINK_VMM_FAKE": "1", **kw}
        out = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=60)
        assert out.returncode == 0, out.stderr
        return int(out.stdout.split()[-1])
    HOST, CUDA, DMABUF = 1, 2, 4
    assert ptr() == HOST                                                         # device buffers not asked for
    assert ptr(FUSELINK_CUDA_PTRS="1") == HOST | CUDA | DMABUF
    assert ptr(FUSELINK_CUDA_PTRS="1", FUSELINK_SOFT_PEERMEM="0") == HOST | CUDA | DMABUF
    assert ptr(FUSELINK_CUDA_PTRS="1", FUSELINK_TRANSPORT="tcp") == HOST | CUDA  # the TCP transport stages device memory itself


def test_verbs_provider_registers_device_memory_by_dmabuf_or_by_address(tmp_path):
    """Through the stand-in libibverbs: without a peer-memory module the provider probes ibv_reg_dmabuf_mr (a descriptor of
    -1 must answer "bad descriptor", not "unsupported") and registers device buffers through it; FUSELINK_PEERMEM=1 (a
    loaded nvidia-peermem) registers them by address; a kernel without dma-buf support and without the module has no
    way to reach device memory and the plugin does not offer NCCL_PTR_CUDA."""
    libdir = _build_fake_ibverbs(tmp_path)
    log = os.path.join(str(tmp_path), "calls.log")
    env = {"FUSELINK_TRANSPORT": "rdma", "LD_LIBRARY_PATH": libdir + ":" + os.environ.get("LD_LIBRARY_PATH", ""), "FUSELINK_FAKE_IB_NDEV": "2",
           "FUSELINK_FAKE_IB_LOG": log, "FUSELINK_CUDA_PTRS": "1", "FUSELINK_VMM_FAKE": "1", "FUSELINK_VMM_FAKE_NGPUS": "2", "FL_HARNESS_VERBOSE": "1",
           "FUSELINK_PEERMEM": "0"}
    tx, rx = _pair([1 << 20, 33], env=env, common=["--device-buffers", "--chunk", "262144"])
    assert tx[0] == 0 and rx[0] == 0, (tx, rx)
    assert _mr_counters(rx[1])[2] == 2 * 2
    calls = open(log).read().splitlines()
    assert sum(l.startswith("reg_dmabuf_mr ") for l in calls) == 2 * 2 * 2          # 2 buffers x 2 devices x 2 processes
    os.remove(log)
    tx, rx = _pair([1 << 20], env=dict(env, FUSELINK_PEERMEM="1"), common=["--device-buffers", "--chunk", "262144"])
    assert tx[0] == 0 and rx[0] == 0 and _mr_counters(rx[1])[2] == 0, (tx, rx)
    assert not any(l.startswith("reg_dmabuf_mr ") for l in open(log).read().splitlines())
    tx, rx = _pair([1 << 20], env=dict(env, FUSELINK_FAKE_IB_DMABUF="0"), common=["--device-buffers", "--chunk", "262144"], timeout=30)
    assert tx[0] != 0 and rx[0] != 0 and "regMr failed" in tx[2] + rx[2], (tx, rx)


def test_enhanced_connection_establishment_is_negotiated(tmp_path):
    """ECE through the stand-in libibverbs: the connecting side offers its options, the accepting side keeps what both
    have and answers with that, the connecting side applies the answer -- all before the queue pairs are connected
    (src/plugin.cc:801-802, 856-857, 986-994).  A library without the calls connects as before."""
    libdir = _build_fake_ibverbs(tmp_path)
    log = os.path.join(str(tmp_path), "calls.log")
    env = {"FUSELINK_TRANSPORT": "rdma", "LD_LIBRARY_PATH": libdir + ":" + os.environ.get("LD_LIBRARY_PATH", ""), "FUSELINK_FAKE_IB_NDEV": "2",
           "FUSELINK_FAKE_IB_LOG": log, "FL_HARNESS_VERBOSE": "1"}
    tx, rx = _pair([1 << 20], env=env, common=["--chunk", "262144"], env_send={"FUSELINK_FAKE_IB_ECE": "0x7"}, env_recv={"FUSELINK_FAKE_IB_ECE": "0xd"})
    assert tx[0] == 0 and rx[0] == 0, (tx, rx)
    sets = [l for l in open(log).read().splitlines() if l.startswith("set_ece ")]
    assert sorted(set(l.split(" ", 2)[2] for l in sets)) == ["given=0x5 kept=0x5", "given=0x7 kept=0x5"]
    assert len(sets) == 2 * 2                                      # one queue pair per device, both ends
    assert "ece offered vendor 0x15b3 options 0x7" in tx[2] and "ece agreed vendor 0x15b3 options 0x5" in rx[2]
    os.remove(log)
    tx, rx = _pair([1 << 20], env=env, common=["--chunk", "262144"], env_send={"FUSELINK_FAKE_IB_ECE": "0x7"})     # the receiver's device has none
    assert tx[0] == 0 and rx[0] == 0, (tx, rx)
    assert not [l for l in open(log).read().splitlines() if l.startswith("set_ece ")]
