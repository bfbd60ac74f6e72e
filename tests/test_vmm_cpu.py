"""cuMem region layer against the memfd/mmap fake driver: the aliasing, export/import and remap semantics
are the ones the CUDA driver gives (same virtual address, new physical backing)."""
import os

import pytest
import torch

from fuselink_b200 import C, have_native

pytestmark = pytest.mark.skipif(not have_native() or torch.cuda.is_available(), reason="CPU-only test of the fake VMM backend")


@pytest.fixture(autouse=True)
def _fake():
    C.vmm_init(1)
    yield


def _view(region, n=1024):
    return C.tensor_from_ptr(C.vmm_ptr(region), [n], torch.int32, -1)


def test_create_slabs_and_usage():
    before = C.vmm_usage(2)
    r = C.vmm_create(2, 5 << 20, 2 << 20)
    assert C.vmm_num_slabs(r) == 3 and C.vmm_size(r) == 6 << 20 and C.vmm_slab_bytes(r) == 2 << 20
    assert C.vmm_usage(2) - before == 6 << 20
    assert [C.vmm_slab_device(r, i) for i in range(3)] == [2, 2, 2]
    assert C.vmm_ptr2dev(C.vmm_ptr(r) + (3 << 20)) == 2 and C.vmm_ptr2dev(12345) == -1
    C.vmm_destroy(r)
    assert C.vmm_usage(2) == before


def test_alias_sees_same_memory():
    r = C.vmm_create(0, 2 << 20, 0)
    a = C.vmm_alias(r, 1)
    _view(r).fill_(11)
    assert (_view(a) == 11).all()
    _view(a)[5] = 99
    assert _view(r)[5] == 99
    C.vmm_destroy(a)
    C.vmm_destroy(r)


def test_export_import_roundtrip():
    r = C.vmm_create(0, 4 << 20, 2 << 20)
    fds = [C.vmm_export_fd(r, i) for i in range(2)]
    imp = C.vmm_import(3, fds, 2 << 20)
    for fd in fds:
        os.close(fd)
    _view(r, 1 << 20).copy_(torch.arange(1 << 20, dtype=torch.int32))
    assert torch.equal(_view(imp, 1 << 20), torch.arange(1 << 20, dtype=torch.int32))
    C.vmm_destroy(imp)
    C.vmm_destroy(r)


def test_remap_keeps_address_and_optionally_contents():
    r = C.vmm_create(0, 4 << 20, 2 << 20)
    ptr = C.vmm_ptr(r)
    old_alias = C.vmm_alias(r, 0)
    _view(r).fill_(7)
    usec = C.vmm_remap_slab(r, 0, 5, True, [0])
    assert usec >= 0 and C.vmm_ptr(r) == ptr
    assert C.vmm_slab_device(r, 0) == 5 and C.vmm_slab_device(r, 1) == 0
    assert (_view(r) == 7).all()                      # contents carried over
    _view(r).fill_(8)
    assert (_view(old_alias) == 7).all()              # the alias still holds the old physical memory
    C.vmm_remap_slab(r, 0, 6, False, [])
    assert C.vmm_slab_device(r, 0) == 6               # fresh backing: contents not carried
    assert C.vmm_usage(6) >= 2 << 20
    C.vmm_destroy(old_alias)
    C.vmm_destroy(r)


def test_dmabuf_descriptor_names_the_memory_mapped_now():
    """The descriptor a NIC registration goes through: it names what is mapped at the address when it is taken, so one
    taken before a re-homing keeps naming the old memory and one taken after names the new."""
    import mmap
    r = C.vmm_create(0, 4 << 20, 2 << 20)
    _view(r, 4096).fill_(21)
    ptr = C.vmm_ptr(r)
    fd_old, off = C.vmm_dmabuf_fd(ptr + 4096, 8192)
    assert off == 4096
    C.vmm_remap_slab(r, 0, 3, True, [0])
    _view(r, 4096).fill_(22)
    fd_new, off_new = C.vmm_dmabuf_fd(ptr + 4096, 8192)
    assert off_new == 4096
    old = mmap.mmap(fd_old, 2 << 20)
    new = mmap.mmap(fd_new, 2 << 20)
    assert int.from_bytes(old[4096:4100], "little") == 21 and int.from_bytes(new[4096:4100], "little") == 22
    new[4096:4100] = (23).to_bytes(4, "little")                     # what a NIC writes through the descriptor ...
    assert _view(r, 4096)[1024] == 23                                     # ... is what the address shows
    old.close(); new.close(); os.close(fd_old); os.close(fd_new)
    fd2, off2 = C.vmm_dmabuf_fd(ptr + (2 << 20) + 100, 64)          # second slab: its own mapping
    assert off2 == 100
    os.close(fd2)
    with pytest.raises(RuntimeError):
        C.vmm_dmabuf_fd(ptr + (2 << 20) - 16, 64)                   # a range that crosses two physical allocations
    C.vmm_destroy(r)


def test_adopt_foreign_allocation_and_rehome():
    owner = C.vmm_create(1, 2 << 20, 0)               # stands in for a buffer another library allocated
    _view(owner).fill_(3)
    adopted = C.vmm_adopt(C.vmm_ptr(owner), 2 << 20, 1)
    C.vmm_remap_slab(adopted, 0, 4, True, [1])        # same VA now backed by "GPU 4", opened to the source GPU
    assert C.vmm_slab_device(adopted, 0) == 4
    assert (_view(owner) == 3).all()
    C.vmm_destroy(adopted)


def test_symmetric_heap_emulated_on_cpu():
    from fuselink_b200.parallel.symm import SymmetricHeap
    heaps = SymmetricHeap.emulated(3, 4 << 20)
    a = [h.alloc_tensor([16], torch.int32) for h in heaps]
    assert len({t.offset for t in a}) == 1
    a[1].local.fill_(5)
    assert (a[0].view_of(1) == 5).all() and (a[0].local == 0).all()
    assert heaps[0].signal_slots("x", 4) == heaps[2].signal_slots("x", 4)
    for h in heaps:
        h.close()


def test_slab_pool_register_remap_release():
    """Pre-created slabs: registering a live buffer re-backs it slab by slab, a single slab can be re-homed without any
    allocation, the old slab returns to its own device's pool, and sizes beyond 2 GiB are plain size_t arithmetic."""
    C.pool_init(4, 6, 2 << 20)
    try:
        sb = C.pool_slab_bytes()
        assert sb == 2 << 20 and [C.pool_free_slabs(d) for d in range(4)] == [6, 6, 6, 6]
        owner = C.vmm_create(1, 3 * sb, 0)                      # someone else's 6 MiB buffer on GPU 1
        view = C.tensor_from_ptr(C.vmm_ptr(owner), [3 * sb // 4], torch.int32, -1)
        view.copy_(torch.arange(3 * sb // 4, dtype=torch.int32))
        r = C.pool_register(C.vmm_ptr(owner), 3 * sb, 1)
        assert C.pool_free_slabs(1) == 3 and C.vmm_num_slabs(r) == 3
        assert torch.equal(view, torch.arange(3 * sb // 4, dtype=torch.int32))       # same address, same bytes
        usec = C.pool_remap(r, 1, 3, True, [1])
        assert usec >= 0 and C.vmm_slab_device(r, 1) == 3 and C.vmm_slab_device(r, 0) == 1
        assert C.pool_free_slabs(3) == 5 and C.pool_free_slabs(1) == 4               # old slab went back to GPU 1's pool
        assert C.vmm_ptr2dev(C.vmm_ptr(r) + sb + 5) == 3
        assert torch.equal(view, torch.arange(3 * sb // 4, dtype=torch.int32))
        C.pool_remap(r, 1, 2, True, [1])                        # second remap takes GPU 2's slab, not the old device's
        assert C.vmm_slab_device(r, 1) == 2 and C.pool_free_slabs(3) == 6 and C.pool_free_slabs(2) == 5
        fresh = C.pool_alloc(0, sb + 1)
        assert C.vmm_num_slabs(fresh) == 2 and C.pool_free_slabs(0) == 4
        with pytest.raises(RuntimeError):
            C.pool_alloc(0, 5 * sb)                             # only 4 slabs left on GPU 0
        C.pool_release(fresh)
        C.pool_release(r)
        assert [C.pool_free_slabs(d) for d in range(4)] == [6, 6, 6, 6]
    finally:
        C.pool_shutdown()


def test_c_library_example_builds_and_runs_without_python(tmp_path):
    """examples/cpp/regions_and_paths.cc against lib/libfuselink.so and include/fuselink.h, on the memfd stand-in."""
    import shutil
    import subprocess
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    lib = os.path.join(root, "fuselink_b200", "lib")
    if not os.path.exists(os.path.join(lib, "libfuselink.so")):
        pytest.skip("libfuselink.so not built")
    cxx = next((c for c in (os.environ.get("CXX"), "g++", "/usr/bin/g++") if c and shutil.which(c)), None)
    if cxx is None:
        pytest.skip("no C++ compiler")
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    exe = str(tmp_path / "regions_and_paths")
    cmd = [cxx, "-std=c++17", "-I", os.path.join(root, "fuselink_b200", "include"), "-I", os.path.join(cuda, "include"),
           os.path.join(root, "examples", "cpp", "regions_and_paths.cc"), "-L", lib, "-lfuselink", f"-Wl,-rpath,{lib}", "-o", exe]
    b = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert b.returncode == 0, b.stderr[-3000:]
    out = subprocess.run([exe, "--fake"], capture_output=True, text=True, timeout=60, env=dict(os.environ, FUSELINK_VMM_FAKE_NGPUS="4"))
    assert out.returncode == 0 and out.stdout.strip().endswith("OK"), out.stdout + out.stderr
    assert "slab 2 now on device 1" in out.stdout and "stripe 0: via path 1" in out.stdout


def test_random_sequences_keep_accounting_and_contents():
    """A long random walk over create / alias / remap (with and without contents) / destroy: the bytes held per device
    always equal the sum over live slabs, addresses never change, and contents survive every keep-contents remap."""
    import random
    rng = random.Random(11)
    base = {d: C.vmm_usage(d) for d in range(8)}
    live = []                                       # (region, slab_bytes, [device per slab], fill value per slab or None)

    def expect_usage():
        u = dict(base)
        for _, sb, devs, _ in live:
            for d in devs:
                u[d] += sb
        return u

    for step in range(300):
        op = rng.random()
        if op < 0.3 or not live:
            dev, nslab = rng.randrange(8), rng.randint(1, 4)
            sb = rng.choice([2 << 20, 4 << 20])
            r = C.vmm_create(dev, nslab * sb, sb)
            live.append((r, sb, [dev] * nslab, [None] * nslab))
        elif op < 0.75:
            r, sb, devs, fills = rng.choice(live)
            s, target, keep = rng.randrange(len(devs)), rng.randrange(8), rng.random() < 0.7
            ptr = C.vmm_ptr(r)
            view = C.tensor_from_ptr(ptr + s * sb, [sb // 4], torch.int32, -1)
            if fills[s] is None or not keep:
                fills[s] = rng.randrange(1 << 30)
                view.fill_(fills[s])
            C.vmm_remap_slab(r, s, target, keep, [devs[0]])
            assert C.vmm_ptr(r) == ptr and C.vmm_slab_device(r, s) == target
            devs[s] = target
            view = C.tensor_from_ptr(ptr + s * sb, [sb // 4], torch.int32, -1)
            if keep:
                assert int(view[0]) == fills[s] and int(view[-1]) == fills[s] and bool((view == fills[s]).all())
            else:
                fills[s] = None
        elif op < 0.85:
            r, sb, devs, fills = rng.choice(live)
            a = C.vmm_alias(r, rng.randrange(8))
            assert C.vmm_size(a) == C.vmm_size(r)
            C.vmm_destroy(a)                            # an alias owns no memory
        else:
            i = rng.randrange(len(live))
            C.vmm_destroy(live.pop(i)[0])
        if step % 10 == 0:
            want = expect_usage()
            assert {d: C.vmm_usage(d) for d in range(8)} == want, step
    while live:
        C.vmm_destroy(live.pop()[0])
    assert {d: C.vmm_usage(d) for d in range(8)} == base
