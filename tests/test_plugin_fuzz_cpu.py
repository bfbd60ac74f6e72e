"""Randomised configurations of the plugin (fixed seeds): transport, number of devices, degree / step / minimum stripe,
queue pairs, adaptive routing, inline, monitor on or off, device buffers (by address or dma-buf), message sizes, chunk size, requests in flight,
channels, threads -- every transfer must be bit exact; and the same with one link broken at a random point, which the
transfer must survive."""
import random

import pytest

from test_plugin_cpu import _pair


def _config(rng):
    transport = rng.choice(["tcp", "rdma"])
    env = {"NCCL_FUSELINK_DEGREE": str(rng.choice([1, 2, 3, 4])), "NCCL_FUSELINK_STEP": str(rng.choice([1, 2, 3])),
           "FUSELINK_MIN_STRIPE_BYTES": str(rng.choice([4096, 65536, 1 << 20])), "FUSELINK_TCP_NDEV": str(rng.choice([1, 2, 4, 8])),
           "FUSELINK_SOFT_NDEV": str(rng.choice([1, 2, 4, 8])), "NCCL_IB_QPS_PER_CONNECTION": str(rng.choice([1, 2, 4])),
           "NCCL_IB_SPLIT_DATA_ON_QPS": str(rng.choice([0, 1])), "NCCL_IB_ADAPTIVE_ROUTING": str(rng.choice([-2, 0, 1])),
           "NCCL_IB_USE_INLINE": str(rng.choice([0, 1])), "FUSELINK_MONITOR": str(rng.choice([0, 1]))}
    if transport == "rdma":
        env.update(FUSELINK_TRANSPORT="rdma", FUSELINK_RDMA_PROVIDER="soft")
    common = ["--chunk", str(rng.choice([4096, 65536, 262144, 1 << 20])), "--inflight", str(rng.choice([1, 2, 8, 32])),
              "--channels", str(rng.choice([1, 1, 2, 4]))]
    if rng.random() < 0.3:
        common.append("--threads")
    if rng.random() < 0.3:
        # device buffers: registered by address or through a dma-buf (the plugin's own descriptor, or one handed in the way
        # NCCL does), at the start of the allocation or inside it
        env.update(FUSELINK_CUDA_PTRS="1", FUSELINK_VMM_FAKE="1", FUSELINK_VMM_FAKE_NGPUS=str(rng.choice([1, 2, 8])),
                   FUSELINK_SOFT_PEERMEM=str(rng.choice([0, 1])), FUSELINK_REMAP=str(rng.choice([0, 1])))
        common.append(rng.choice(["--device-buffers", "--device-buffers", "--nccl-dmabuf"]))
        common += ["--reg-offset", str(rng.choice([0, 0, 256, 4096]))]
    sizes = [rng.choice([0, 1, 17, 4096, 4097, 65536, 1 << 20, (1 << 20) + 3, 5 << 20]) for _ in range(rng.randint(1, 4))]
    return env, common, sizes


@pytest.mark.parametrize("seed", range(10))
def test_random_configuration_is_bit_exact(seed):
    env, common, sizes = _config(random.Random(1000 + seed))
    tx, rx = _pair(sizes, env=env, common=common, timeout=120)
    assert tx[0] == 0 and rx[0] == 0, (env, common, sizes, tx, rx)


@pytest.mark.parametrize("seed", range(10))
def test_random_link_failure_is_survived(seed):
    rng = random.Random(2000 + seed)
    transport = rng.choice(["tcp", "rdma"])
    ndev = rng.choice([2, 4, 8])
    env = {"NCCL_FUSELINK_DEGREE": str(rng.choice([1, 2, 3])), "FUSELINK_MIN_STRIPE_BYTES": "65536", "FUSELINK_TCP_NDEV": str(ndev),
           "FUSELINK_SOFT_NDEV": str(ndev), "NCCL_IB_QPS_PER_CONNECTION": str(rng.choice([1, 2])), "FUSELINK_NET_TIMEOUT_MS": "8000",
           "FUSELINK_MONITOR": str(rng.choice([0, 1]))}
    after = rng.choice([1000, 300000, 1 << 20, 3 << 20, 7 << 20])
    env_send, env_recv = {}, {}
    if transport == "rdma":
        env.update(FUSELINK_TRANSPORT="rdma", FUSELINK_RDMA_PROVIDER="soft")
        who = rng.choice(["send", "recv"])
        fault = {"FUSELINK_SOFT_FAULT_DEV": str(rng.randrange(ndev)),
                 "FUSELINK_SOFT_FAULT_AFTER_BYTES": str(after if who == "send" else rng.choice([200, 1500, 5000]))}
        (env_send if who == "send" else env_recv).update(fault)
    else:
        env_send["FUSELINK_FAULT_CLOSE_AFTER_BYTES"] = str(after)
    sizes = [rng.choice([1 << 20, 5 << 20, 12 << 20]) for _ in range(rng.randint(1, 3))] + [7]
    common = ["--chunk", str(rng.choice([65536, 262144, 1 << 20])), "--inflight", str(rng.choice([1, 4, 8]))]
    tx, rx = _pair(sizes, env=env, common=common, timeout=120, env_send=env_send, env_recv=env_recv)
    assert tx[0] == 0 and rx[0] == 0, (env, env_send, env_recv, common, sizes, tx, rx)
