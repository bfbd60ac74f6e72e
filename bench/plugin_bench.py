#!/usr/bin/env python
"""Throughput of the ncclNet plugin on the host, without GPUs or NCCL: two processes per connection drive the plugin's
entry points through ``fl_net_harness`` over loopback.  One JSON line per measurement; the rate is that of the
post/test loops alone (payload generation and the bitwise compare are outside).

    python bench/plugin_bench.py                 # transports, striping over rate-limited NICs, two-job contention
    python bench/plugin_bench.py --sections nic  # one section: transports | nic | contention
"""
import argparse
import json
import os
import subprocess
import tempfile
import uuid

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB = os.path.join(ROOT, "fuselink_b200", "lib")
HARNESS, PLUGIN, MONITOR = (os.path.join(LIB, n) for n in ("fl_net_harness", "libnccl-net-fuselink.so", "fuselink-monitor"))


def rate(out: str) -> float:
    line = [l for l in out.splitlines() if l.startswith("OK ")][0]
    return float(line.split("(")[2].split()[0])


def pairs(n_jobs: int, size: int, env: dict, common) -> list:
    """n_jobs sender/receiver pairs at the same time; GB/s seen by each receiver."""
    procs, dirs = [], []
    try:
        for _ in range(n_jobs):
            d = tempfile.mkdtemp()
            dirs.append(d)
            hf = os.path.join(d, "handle")
            e = dict(os.environ, NCCL_SOCKET_IFNAME="lo", **env)
            args = [*common, str(size)]
            rx = subprocess.Popen([HARNESS, PLUGIN, "recv", hf, *args], env=e, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
            tx = subprocess.Popen([HARNESS, PLUGIN, "send", hf, *args], env=e, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
            procs.append((tx, rx))
        out = []
        for tx, rx in procs:
            tx.communicate(timeout=600)
            rxo, rxe = rx.communicate(timeout=600)
            if tx.returncode or rx.returncode:
                raise RuntimeError(rxe[-2000:])
            out.append(rate(rxo))
        return out
    finally:
        import shutil
        for tx, rx in procs:
            for p in (tx, rx):
                if p.poll() is None:
                    p.kill()
        for d in dirs:
            shutil.rmtree(d, ignore_errors=True)


def emit(**kw):
    print(json.dumps(kw), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--sections", default="transports nic contention")
    ap.add_argument("--size-mib", type=int, default=1024)
    a = ap.parse_args()
    chunk = ["--chunk", "524288", "--inflight", "8"]
    soft = {"FUSELINK_TRANSPORT": "rdma", "FUSELINK_RDMA_PROVIDER": "soft"}
    many = {"FUSELINK_TCP_NDEV": "8", "FUSELINK_SOFT_NDEV": "8", "NCCL_FUSELINK_DEGREE": "2", "FUSELINK_MIN_STRIPE_BYTES": "65536"}
    if "transports" in a.sections:
        big, small = a.size_mib << 20, (a.size_mib << 20) // 4
        for name, env, common, size in [
            ("tcp, 1 connection", {}, chunk, big),
            ("tcp, 4 connections x 2 stripes, one thread", many, ["--channels", "4", *chunk], big),
            ("tcp, 4 connections, one thread each", many, ["--channels", "4", "--threads", *chunk], small),
            ("rdma over the software NIC, 1 connection", soft, chunk, big),
            ("rdma over the software NIC, 4 connections, one thread each", dict(soft, **many), ["--channels", "4", "--threads", *chunk], small),
        ]:
            emit(section="transports", config=name, bytes=size, GBps=pairs(1, size, env, common)[0])
    if "nic" in a.sections:
        for degree in (1, 2, 4, 8):
            env = {"FUSELINK_TCP_NDEV": "8", "FUSELINK_TCP_NIC_MBPS": "200", "NCCL_FUSELINK_DEGREE": str(degree), "FUSELINK_MIN_STRIPE_BYTES": "65536"}
            emit(section="nic", config=f"8 NICs of 200 MB/s, degree {degree}", GBps=pairs(1, 192 << 20, env, ["--chunk", "1048576", "--inflight", "8"])[0])
    if "contention" in a.sections:
        tag = uuid.uuid4().hex[:10]
        nic_shm, mon_shm = f"/fl_nic_{tag}", f"/fl_mon_{tag}"
        base = {"FUSELINK_TCP_NDEV": "8", "FUSELINK_TCP_NIC_MBPS": "200", "FUSELINK_TCP_NIC_SHM": nic_shm, "NCCL_FUSELINK_DEGREE": "1"}
        common = ["--chunk", "1048576", "--inflight", "8"]
        daemon = None
        try:
            emit(section="contention", config="two jobs, no monitor", GBps=pairs(2, 96 << 20, dict(base, FUSELINK_MONITOR="0"), common))
            daemon = subprocess.Popen([MONITOR, "--shm", mon_shm, "--groups", "8", "--seconds", "600"], stdout=subprocess.PIPE, text=True)
            daemon.stdout.readline()
            shared = dict(base, FUSELINK_MONITOR_SHM=mon_shm)
            emit(section="contention", config="two jobs, shared monitor", GBps=pairs(2, 96 << 20, shared, common))
            emit(section="contention", config="two jobs, shared monitor, degree 2",
                 GBps=pairs(2, 96 << 20, dict(shared, NCCL_FUSELINK_DEGREE="2", FUSELINK_MIN_STRIPE_BYTES="65536"), common))
        finally:
            if daemon is not None:
                daemon.terminate()
            for n in (nic_shm, mon_shm):
                try:
                    os.unlink("/dev/shm" + n)
                except OSError:
                    pass


if __name__ == "__main__":
    main()
