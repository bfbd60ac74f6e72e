"""The ncclNet plugin loaded by a real NCCL: two ranks on two GPUs exchange messages with NCCL's send/recv while NCCL's
intra-node transports are switched off, so every byte goes proxy thread -> plugin -> TCP transport -> plugin -> proxy
thread.  This is the reference's one documented way of use (README.md:37-42: NCCL_NET_PLUGIN=fuselink plus the library
on the loader path) and its bandwidth experiment in miniature (experiments/bw_test/run_bw_test.sbatch:29-50).

The run fails unless NCCL's own log names the plugin, the plugin's counters show that receives went through its path
selector, and every received byte is right."""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(extra_env, args, port, limit_s=420):
    lib = os.path.join(ROOT, "fuselink_b200", "lib")
    env = dict(os.environ, NCCL_NET_PLUGIN="fuselink", LD_LIBRARY_PATH=lib + ":" + os.environ.get("LD_LIBRARY_PATH", ""),
               NCCL_DEBUG="INFO", NCCL_DEBUG_SUBSYS="INIT,NET", NCCL_NVLS_ENABLE="0", **extra_env)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(ROOT, "bench", "nccl_plugin_sendrecv.py"), *args]
    try:
        out = subprocess.run(cmd, capture_output=True, text=True, timeout=limit_s, env=env)
    except subprocess.TimeoutExpired as e:       # show how far the run got: NCCL's and the plugin's log lines
        def tail(b):
            return (b.decode(errors="replace") if isinstance(b, bytes) else (b or ""))[-6000:]
        raise AssertionError(f"no result within {limit_s} s\n--- stdout\n{tail(e.stdout)}\n--- stderr\n{tail(e.stderr)}") from None
    text = out.stdout + out.stderr
    assert out.returncode == 0, text[-6000:]
    rows = [json.loads(l) for l in out.stdout.splitlines() if l.startswith("{")]
    assert rows, text[-3000:]
    return rows[-1], text


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs >= 2 GPUs")
def test_nccl_sendrecv_goes_through_the_plugin():
    """4 KiB to 64 MiB in powers of two, host-staged (the plugin's default: it reports host pointer support, so NCCL's
    proxy hands it pinned host buffers)."""
    res, text = _run({}, ["--size-lo", "12", "--size-hi", "26", "--iters", "3", "--warmup", "1"], 29671)
    assert "FuseLink" in text, "NCCL's log does not name the plugin:\n" + text[-3000:]
    assert res["plugin_selector_decisions"] > 0
    assert [r["bytes"] for r in res["results"]] == [1 << k for k in range(12, 27)]


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs >= 2 GPUs")
def test_striping_under_the_proxy_adds_the_virtual_nics_bandwidth():
    """The TCP transport's four virtual NICs held to 300 MB/s each: with NCCL_FUSELINK_DEGREE=1 a message gets one NIC, with 4 it gets the sum
    (the reference's mechanism, under NCCL's own proxy thread and chunking)."""
    rates = {}
    for degree, port in ((1, 29673), (4, 29675)):
        res, _ = _run({"FUSELINK_TCP_NIC_MBPS": "300", "NCCL_FUSELINK_DEGREE": str(degree),
                       "NCCL_NCHANNELS_PER_NET_PEER": "1", "NCCL_MIN_NCHANNELS": "1", "NCCL_MAX_NCHANNELS": "1"},
                      ["--size-lo", "25", "--size-hi", "25", "--iters", "3", "--warmup", "1"], port)
        rates[degree] = res["results"][0]["GBps_per_direction"]
    assert rates[4] > 2.0 * rates[1], rates

