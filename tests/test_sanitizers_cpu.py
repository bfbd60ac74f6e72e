"""Sanitizer tier of the host-side code: the plugin and its two-process harness built with AddressSanitizer +
UndefinedBehaviorSanitizer move data without a report, and the lock-free monitor survives a multi-threaded stress run under
ThreadSanitizer (and under ASan/UBSan) with its exclusivity invariant intact."""
import os
import subprocess
import sys
import tempfile

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def _build(kind):
    from fuselink_b200 import build
    try:
        return build.build_sanitized(kind)
    except RuntimeError as e:
        pytest.skip(f"sanitizer build not available here: {str(e)[:200]}")


TRANSPORTS = {
    "tcp": {},
    "tcp-direct": {"FUSELINK_CUDA_PTRS": "1", "FUSELINK_VMM_FAKE": "1", "FUSELINK_VMM_FAKE_NGPUS": "4"},
    "rdma-soft": {"FUSELINK_TRANSPORT": "rdma", "FUSELINK_RDMA_PROVIDER": "soft", "NCCL_IB_QPS_PER_CONNECTION": "2"},
    # device buffers, re-homed, registered through dma-buf descriptors (the software NIC maps them itself)
    "rdma-dmabuf": {"FUSELINK_TRANSPORT": "rdma", "FUSELINK_RDMA_PROVIDER": "soft", "FUSELINK_SOFT_PEERMEM": "0", "FUSELINK_CUDA_PTRS": "1",
                    "FUSELINK_VMM_FAKE": "1", "FUSELINK_VMM_FAKE_NGPUS": "4"},
}


@pytest.mark.parametrize("transport", list(TRANSPORTS))
def test_plugin_transfer_under_asan_ubsan(transport):
    art = _build("address,undefined")
    with tempfile.TemporaryDirectory() as d:
        hf = os.path.join(d, "h")
        env = dict(os.environ, NCCL_SOCKET_IFNAME="lo", ASAN_OPTIONS="detect_leaks=1:abort_on_error=1", UBSAN_OPTIONS="halt_on_error=1",
                   NCCL_FUSELINK_DEGREE="3", FUSELINK_MIN_STRIPE_BYTES="4096", **TRANSPORTS[transport])
        sizes = ["0", "4097", str(1 << 20), str(5 << 20)]
        if transport in ("tcp-direct", "rdma-dmabuf"):
            sizes = ["--device-buffers"] + sizes
        rx = subprocess.Popen([art["harness"], art["plugin"], "recv", hf, "--chunk", "262144", *sizes], env=env, stdout=subprocess.PIPE,
                              stderr=subprocess.PIPE, text=True)
        tx = subprocess.Popen([art["harness"], art["plugin"], "send", hf, "--chunk", "262144", *sizes], env=env, stdout=subprocess.PIPE,
                              stderr=subprocess.PIPE, text=True)
        txo, txe = tx.communicate(timeout=180)
        rxo, rxe = rx.communicate(timeout=180)
    assert tx.returncode == 0 and rx.returncode == 0, (txo, txe[-2000:], rxo, rxe[-2000:])
    assert "ERROR: AddressSanitizer" not in txe + rxe and "runtime error" not in txe + rxe
    assert "LeakSanitizer" not in txe + rxe, (txe[-2000:], rxe[-2000:])       # every connection, request and mapping is given back


@pytest.mark.parametrize("transport", ["tcp", "rdma-soft"])
def test_threaded_plugin_under_tsan(transport):
    """Four proxy-like threads per process drive four connections through the plugin built with ThreadSanitizer: the
    shared state (channel counter, selector, monitor table, registration table, software NIC) must be race-free."""
    art = _build("thread")
    with tempfile.TemporaryDirectory() as d:
        hf = os.path.join(d, "h")
        env = dict(os.environ, NCCL_SOCKET_IFNAME="lo", TSAN_OPTIONS="halt_on_error=1", NCCL_FUSELINK_DEGREE="2",
                   FUSELINK_MIN_STRIPE_BYTES="4096", **TRANSPORTS[transport])
        args = ["--channels", "4", "--threads", "--chunk", "131072", "--inflight", "4", str(2 << 20), "4097"]
        rx = subprocess.Popen([art["harness"], art["plugin"], "recv", hf, *args], env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
        tx = subprocess.Popen([art["harness"], art["plugin"], "send", hf, *args], env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
        txo, txe = tx.communicate(timeout=300)
        rxo, rxe = rx.communicate(timeout=300)
    assert "WARNING: ThreadSanitizer" not in txe + rxe, (txe[-3000:], rxe[-3000:])
    assert tx.returncode == 0 and rx.returncode == 0, (txo, txe[-2000:], rxo, rxe[-2000:])


@pytest.mark.parametrize("kind", ["thread", "address,undefined"])
def test_monitor_stress_under_sanitizer(kind):
    art = _build(kind)
    env = dict(os.environ, TSAN_OPTIONS="halt_on_error=1", ASAN_OPTIONS="detect_leaks=0", UBSAN_OPTIONS="halt_on_error=1")
    out = subprocess.run([art["monitor_stress"], "4000"], env=env, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, (out.stdout, out.stderr[-3000:])
    assert "violations 0" in out.stdout
    assert "WARNING: ThreadSanitizer" not in out.stderr
