"""The cuMem region layer on the CUDA driver: a buffer keeps its virtual address while the physical memory behind it moves
(to fresh memory on the same GPU, and with two GPUs to the other GPU and back), an allocation made by someone else is taken
over and re-homed, the slab pool re-backs single slabs, and the layer's usage count returns to where it started.

Every step is a synchronous driver call; nothing reads a range between its unmap and its map (the stream is drained before
each remap).  What the reference does once per registered buffer (src/fuselink.cc:20-56) and times in its unused helper
(src/plugin.cc:1139-1163: "Remap time") is `vmm_remap_slab` here; the printed microseconds are that measurement."""
import pytest
import torch

pytestmark = pytest.mark.gpu

MB = 1 << 20


@pytest.fixture(scope="module")
def C():
    from fuselink_b200 import C as ext
    torch.cuda.init()
    torch.zeros(1, device="cuda:0")
    ext.vmm_init(0)
    return ext


def _view(C, region, n, device=0):
    return C.tensor_from_ptr(C.vmm_ptr(region), [n], torch.int32, device)


def _pattern(n, seed):
    return torch.arange(n, dtype=torch.int32, device="cuda:0") * 7 + seed


def test_remap_on_one_gpu_keeps_address_and_contents(C):
    before = C.vmm_usage(0)
    r = C.vmm_create(0, 8 * MB, 2 * MB)
    nslab = C.vmm_num_slabs(r)
    sb = C.vmm_slab_bytes(r)
    assert nslab * sb == C.vmm_size(r) >= 8 * MB and C.vmm_usage(0) - before == C.vmm_size(r)
    n = C.vmm_size(r) // 4
    ptr = C.vmm_ptr(r)
    v = _view(C, r, n)
    v.copy_(_pattern(n, 3))
    torch.cuda.synchronize()
    usec = C.vmm_remap_slab(r, 0, 0, True, [0])            # new physical memory on the same GPU, contents carried
    assert C.vmm_ptr(r) == ptr and C.vmm_slab_device(r, 0) == 0 and usec > 0
    assert torch.equal(_view(C, r, n), _pattern(n, 3))
    assert C.vmm_usage(0) - before == C.vmm_size(r)       # the old slab was released
    usec2 = C.vmm_remap_slab(r, nslab - 1, 0, False, [0])  # fresh backing, contents not carried: the rest is untouched
    keep = (nslab - 1) * sb // 4
    assert torch.equal(_view(C, r, n)[:keep], _pattern(n, 3)[:keep])
    _view(C, r, n)[keep:].fill_(5)
    torch.cuda.synchronize()
    print(f"remap of a {sb >> 20} MiB slab on one GPU: {usec} us with the copy, {usec2} us without")
    assert C.vmm_ptr2dev(ptr + sb + 64) == 0
    C.vmm_destroy(r)
    assert C.vmm_usage(0) == before


def test_alias_and_export_import_see_the_same_memory(C):
    import os
    r = C.vmm_create(0, 4 * MB, 2 * MB)
    n = C.vmm_size(r) // 4
    a = C.vmm_alias(r, 0)
    _view(C, r, n).copy_(_pattern(n, 11))
    torch.cuda.synchronize()
    assert torch.equal(_view(C, a, n), _pattern(n, 11))
    fds = [C.vmm_export_fd(r, i) for i in range(C.vmm_num_slabs(r))]
    imp = C.vmm_import(0, fds, C.vmm_slab_bytes(r))
    for fd in fds:
        os.close(fd)
    _view(C, imp, n)[:16].fill_(-1)
    torch.cuda.synchronize()
    assert bool((_view(C, r, n)[:16] == -1).all()) and torch.equal(_view(C, a, n)[16:], _pattern(n, 11)[16:])
    for x in (imp, a, r):
        C.vmm_destroy(x)


def test_adopting_an_allocation_made_elsewhere(C):
    """A cuMemCreate allocation this layer did not make (as NCCL's staging buffers are with NCCL_CUMEM_ENABLE=1) is taken
    over by address and re-homed; its owner keeps using the same pointer and frees it as usual afterwards."""
    cu = pytest.importorskip("cuda.bindings.driver")

    def ok(res):
        assert int(res[0]) == 0, res
        return res[1] if len(res) > 1 else None

    prop = cu.CUmemAllocationProp()
    prop.type = cu.CUmemAllocationType.CU_MEM_ALLOCATION_TYPE_PINNED
    prop.location.type = cu.CUmemLocationType.CU_MEM_LOCATION_TYPE_DEVICE
    prop.location.id = 0
    prop.requestedHandleTypes = cu.CUmemAllocationHandleType.CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR
    gran = ok(cu.cuMemGetAllocationGranularity(prop, cu.CUmemAllocationGranularity_flags.CU_MEM_ALLOC_GRANULARITY_RECOMMENDED))
    size = 2 * gran
    h = ok(cu.cuMemCreate(size, prop, 0))
    va = ok(cu.cuMemAddressReserve(size, gran, 0, 0))
    ok(cu.cuMemMap(va, size, 0, h, 0))
    desc = cu.CUmemAccessDesc()
    desc.location.type = cu.CUmemLocationType.CU_MEM_LOCATION_TYPE_DEVICE
    desc.location.id = 0
    desc.flags = cu.CUmemAccess_flags.CU_MEM_ACCESS_FLAGS_PROT_READWRITE
    ok(cu.cuMemSetAccess(va, size, [desc], 1))
    n = size // 4
    mine = C.tensor_from_ptr(int(va), [n], torch.int32, 0)
    mine.copy_(_pattern(n, 23))
    torch.cuda.synchronize()
    target = 1 if torch.cuda.device_count() > 1 else 0
    if target:
        torch.zeros(1, device="cuda:1")
    before, before_t = C.vmm_usage(0), C.vmm_usage(target)
    r = C.vmm_adopt(int(va), size, 0)
    assert C.vmm_ptr(r) == int(va) and C.vmm_num_slabs(r) == 1 and C.vmm_usage(0) == before
    usec = C.vmm_remap_slab(r, 0, target, True, [0] if target == 0 else [0, 1])
    assert C.vmm_slab_device(r, 0) == target and C.vmm_ptr2dev(int(va)) == target
    assert torch.equal(mine, _pattern(n, 23))              # the owner's pointer, now backed by memory this layer created
    mine.add_(1)
    torch.cuda.synchronize()
    assert torch.equal(mine, _pattern(n, 24))
    assert C.vmm_usage(target) - before_t >= size
    print(f"adopted {size >> 20} MiB allocation re-homed onto GPU {target}: {usec} us")
    C.vmm_destroy(r)                                       # drops this layer's reference; the mapping stays the owner's to undo
    assert C.vmm_usage(target) == before_t
    ok(cu.cuMemUnmap(va, size))
    ok(cu.cuMemRelease(h))
    ok(cu.cuMemAddressFree(va, size))


def test_slab_pool_rebacks_single_slabs(C):
    nd = min(torch.cuda.device_count(), 2)
    before = [C.vmm_usage(d) for d in range(nd)]
    C.pool_init(nd, 8, 2 * MB)
    try:
        sb = C.pool_slab_bytes()
        assert C.pool_free_slabs(0) == 8
        r = C.pool_alloc(0, 3 * sb)
        assert C.pool_free_slabs(0) == 5 and C.vmm_num_slabs(r) == 3
        n = 3 * sb // 4
        v = _view(C, r, n)
        v.copy_(_pattern(n, 31))
        torch.cuda.synchronize()
        target = nd - 1
        usec = C.pool_remap(r, 1, target, True, [0] if target == 0 else [0, 1])
        assert C.vmm_slab_device(r, 1) == target and C.vmm_slab_device(r, 0) == 0
        assert torch.equal(_view(C, r, n), _pattern(n, 31))
        assert C.pool_free_slabs(0) == (5 if target == 0 else 6)            # the old slab went back to its pool
        print(f"pool remap of one {sb >> 20} MiB slab to GPU {target} (no allocation on the way): {usec} us")
        C.pool_release(r)
        assert C.pool_free_slabs(0) == 8 and (nd == 1 or C.pool_free_slabs(1) == 8)
    finally:
        C.pool_shutdown()
    assert [C.vmm_usage(d) for d in range(nd)] == before


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs >= 2 GPUs")
def test_rehoming_onto_the_other_gpu_and_back(C):
    """The reference's trick on real memory: the buffer's address stays, its bytes now live on GPU 1, and a kernel on GPU 0
    reads and writes them through the same pointer (over NVLink); then the buffer goes home again."""
    torch.zeros(1, device="cuda:1")
    u0, u1 = C.vmm_usage(0), C.vmm_usage(1)
    r = C.vmm_create(0, 64 * MB, 0)                        # one slab: the whole buffer moves, as in the reference
    size = C.vmm_size(r)
    n = size // 4
    ptr = C.vmm_ptr(r)
    v = _view(C, r, n)
    v.copy_(_pattern(n, 41))
    torch.cuda.synchronize()
    away = C.vmm_remap_slab(r, 0, 1, True, [0, 1])
    assert C.vmm_ptr(r) == ptr and C.vmm_slab_device(r, 0) == 1 and C.vmm_ptr2dev(ptr + 4096) == 1
    assert C.vmm_usage(1) - u1 == size and C.vmm_usage(0) == u0
    # GPU 0 kernels through the same address (this library's copy kernel, launched on GPU 0; PyTorch itself refuses to wrap
    # the pointer as a cuda:0 tensor because the driver now reports GPU 1 as its home -- which is the point)
    def gpu0_copy(dst_addr, src_addr, nbytes):
        with torch.cuda.device(0):
            C.put_chunks([(src_addr, dst_addr, nbytes, 0, 0, 0)], 1 << 20, 0, False, 64, 512, 0)
            torch.cuda.synchronize()

    got = torch.empty(n, dtype=torch.int32, device="cuda:0")
    gpu0_copy(got.data_ptr(), ptr, size)
    assert torch.equal(got, _pattern(n, 41))
    twice = _pattern(n, 41) * 2
    gpu0_copy(ptr, twice.data_ptr(), size)                 # GPU 0 writes through the pointer, over NVLink
    on1 = C.tensor_from_ptr(ptr, [n], torch.int32, 1)      # and GPU 1 sees it in what is now its own memory
    with torch.cuda.device(1):
        assert torch.equal(on1.to("cuda:0"), twice)
        torch.cuda.synchronize()
    home = C.vmm_remap_slab(r, 0, 0, True, [0])
    assert C.vmm_slab_device(r, 0) == 0 and C.vmm_usage(1) == u1 and C.vmm_usage(0) - u0 == size
    assert torch.equal(_view(C, r, n), _pattern(n, 41) * 2)
    # the reference's "Remap time": a few more round trips now that the driver has seen every call once
    aways, homes, bares = [], [], []
    for _ in range(5):
        aways.append(C.vmm_remap_slab(r, 0, 1, True, [0, 1]))
        homes.append(C.vmm_remap_slab(r, 0, 0, True, [0]))
    assert torch.equal(_view(C, r, n), _pattern(n, 41) * 2)
    for _ in range(5):
        bares.append(C.vmm_remap_slab(r, 0, 1, False, [0, 1]))
        bares.append(C.vmm_remap_slab(r, 0, 0, False, [0]))
    torch.cuda.synchronize()
    med = lambda v: sorted(v)[len(v) // 2]
    print(f"re-homing {size >> 20} MiB (median of 5 after the first): to GPU 1 {med(aways)} us, home {med(homes)} us (both carry the "
          f"contents), without the copy {med(bares)} us; first calls {away} / {home} us")
    C.vmm_remap_slab(r, 0, 1, False, [0, 1])
    C.vmm_destroy(r)
    assert C.vmm_usage(0) == u0 and C.vmm_usage(1) == u1
