"""Peer-copy kernels on one GPU: `world` virtual ranks share the device, every peer address is local, and
ranks are run one after the other (a kernel that waits is launched only after its producers)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture()
def heaps():
    from fuselink_b200.parallel.symm import SymmetricHeap
    hs = SymmetricHeap.emulated(4, 96 << 20)
    yield hs
    for h in hs:
        h.close()


@pytest.mark.parametrize("engine", ["ldst", "bulk"])
@pytest.mark.parametrize("nbytes", [16, 1000, 4096 + 48, 1 << 20, (8 << 20) + 16])
def test_put_and_wait(heaps, engine, nbytes):
    from fuselink_b200.ops.comm import Channel
    chans = [Channel(h, "t", engine=engine) for h in heaps]
    dst = [h.alloc_tensor([nbytes + 64], torch.uint8) for h in heaps]
    src = torch.randint(0, 255, (nbytes,), dtype=torch.uint8, device="cuda")
    chans[0].put(src, 2, dst[0].offset + 16)
    chans[2].expect(0, nbytes)
    chans[2].wait()
    torch.cuda.synchronize()
    heaps[2].check_status()
    got = dst[2].local
    assert torch.equal(got[16:16 + nbytes], src)
    assert (got[:16] == 0).all() and (got[16 + nbytes:] == 0).all()


def test_unaligned_put(heaps):
    from fuselink_b200.ops.comm import Channel
    chans = [Channel(h, "u") for h in heaps]
    dst = [h.alloc_tensor([5000], torch.uint8) for h in heaps]
    src = torch.randint(0, 255, (4001,), dtype=torch.uint8, device="cuda")
    chans[1].put(src[1:], 3, dst[0].offset + 3)
    chans[3].expect(1, 4000)
    chans[3].wait()
    torch.cuda.synchronize()
    assert torch.equal(dst[3].local[3:4003], src[1:])


@pytest.mark.parametrize("engine", ["ldst", "bulk"])
def test_all_to_all(heaps, engine):
    from fuselink_b200.ops.comm import Channel, all_to_all
    W, n = 4, 300_000
    chans = [Channel(h, "a2a", engine=engine) for h in heaps]
    recv = [h.alloc_tensor([W, n], torch.float32) for h in heaps]
    send = [torch.randn(W, n, device="cuda") for _ in range(W)]
    for r in range(W):
        all_to_all(chans[r], send[r], recv[r], wait=False)
    for r in range(W):
        chans[r].wait()
    torch.cuda.synchronize()
    for r in range(W):
        heaps[r].check_status()
        for s in range(W):
            assert torch.equal(recv[r].local[s], send[s][r])


def test_barrier_and_timeout_status(heaps):
    from fuselink_b200.ops.comm import barrier
    for h in heaps:
        barrier(h, "b", signal=True, wait=False)
    for h in heaps:
        barrier(h, "b", signal=False, wait=True)
    torch.cuda.synchronize()
    for h in heaps:
        h.check_status()


def test_striped_relay(heaps):
    from fuselink_b200.ops.comm import StripedP2P
    from fuselink_b200 import C
    nbytes = 24 << 20
    sp = [StripedP2P(h, "s", 16 << 20) for h in heaps]
    dst = [h.alloc_tensor([nbytes], torch.uint8) for h in heaps]
    src = torch.randint(0, 255, (nbytes,), dtype=torch.uint8, device="cuda")
    mon = C.monitor_open("", True, 4, 1, 160)
    stripes = C.select_paths(mon, 3, 1, 1 << 20, 512 * 1024, True, 0, 1, nbytes, 0, C.monitor_now_ns())
    assert len(stripes) == 3 and sum(b for _, _, b in stripes) == nbytes
    # source first, then the relays, then the destination: each waits only on what already ran
    order = [0] + [p for p, _, _ in stripes if p != 1] + [1]
    for r in order:
        sp[r].transfer(0, 1, src if r == 0 else None, dst[r], nbytes, stripes)
    torch.cuda.synchronize()
    for h in heaps:
        h.check_status()
    assert torch.equal(dst[1].local, src)
    C.monitor_close(mon, False)
