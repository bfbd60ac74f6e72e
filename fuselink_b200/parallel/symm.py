"""Symmetric heap: one cuMem region per rank, mapped read/write by every GPU of the box.

Every rank creates a physical allocation with ``cuMemCreate`` (through the native region layer), exports it
as a POSIX file descriptor, hands the descriptor to every peer over a Unix-domain socket (``SCM_RIGHTS``),
and maps every peer's allocation into its own address space.  After that ``heap.addr(off, rank=r)`` is an
address a kernel running on this GPU can load from / store to, and it refers to byte ``off`` of rank r's
region.  This is the reference's buffer-remapping idea (src/fuselink.cc:20-56: per-GPU physical
allocations + alias VAs) turned inside out: instead of re-pointing one VA at a relay GPU, every buffer is
addressable from everywhere, and kernels choose the path.

The first ``SIGNAL_BYTES`` of each region are the rank's *signal pad*: monotone uint32 words that peers
write with release semantics and the owner polls with acquire semantics (see csrc/kernels/comm_kernels.cuh).

``SymmetricHeap.emulated(world, ...)`` builds ``world`` regions on ONE GPU inside one process.  All "peer"
addresses are then local, which lets every multi-rank code path be exercised rank after rank on a single
GPU (kernels that wait on other ranks must then only be launched after their producers).
"""
from __future__ import annotations

import os
import socket
import threading
import uuid
from typing import List, Optional, Sequence

import torch

from .._ext import require_native

SIGNAL_BYTES = 256 * 1024          # 65536 uint32 words
STATUS_BYTES = 256                 # int32 status block(s) written by kernels on a timed-out wait
_ALIGN = 256


def _round_up(x: int, a: int) -> int:
    return (x + a - 1) // a * a


class SymmetricHeap:
    def __init__(self, rank: int, world: int, device: int, size: int, regions: Sequence[int], bases: Sequence[int],
                 shared_state: Optional[dict] = None):
        self.C = require_native()
        self.rank, self.world, self.device, self.size = rank, world, device, size
        self._regions = list(regions)      # native handles owned by this object (own + imported)
        self.base: List[int] = list(bases)  # base[r]: address of rank r's region as mapped in this process
        # allocator / sequence state is shared between the virtual ranks of an emulated world
        self._state = shared_state if shared_state is not None else {"bump": SIGNAL_BYTES + STATUS_BYTES, "seq": {}, "slots": {}, "next_slot": 0}
        self._closed = False

    # ------------------------------------------------------------------ construction
    @classmethod
    def create(cls, size: int, group=None, device: Optional[int] = None) -> "SymmetricHeap":
        """Collective over ``group`` (default: the world group): one region per rank, all mapped everywhere.

        On a machine without a GPU (or with ``device=-1``) the regions are memfd-backed host memory shared between the
        processes the same way -- file descriptors over SCM_RIGHTS -- which is what multi-process CPU tests run on."""
        import torch.distributed as dist

        C = require_native()
        on_gpu = torch.cuda.is_available() and (device is None or device >= 0)
        if on_gpu:
            if device is None:
                device = torch.cuda.current_device()
            torch.cuda.set_device(device)
            torch.cuda.init()
            torch.zeros(1, device=f"cuda:{device}")  # make sure the primary context exists and is current
            C.vmm_init(0)
        else:
            device = -1
            C.vmm_init(1)
        vdev = max(device, 0)
        rank = dist.get_rank(group) if dist.is_initialized() else 0
        world = dist.get_world_size(group) if dist.is_initialized() else 1
        gran = C.vmm_granularity(vdev)
        size = _round_up(max(size, SIGNAL_BYTES + STATUS_BYTES + _ALIGN), gran)
        mine = C.vmm_create(vdev, size, 0)
        regions = [None] * world
        bases = [0] * world
        regions[rank] = mine
        bases[rank] = C.vmm_ptr(mine)
        if world > 1:
            fd = C.vmm_export_fd(mine, 0)
            token = [uuid.uuid4().hex if rank == 0 else None]
            dist.broadcast_object_list(token, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
            fds = _exchange_fds(token[0], rank, world, fd, lambda: dist.barrier(group=group))
            os.close(fd)
            for r in range(world):
                if r == rank:
                    continue
                imp = C.vmm_import(vdev, [fds[r]], size)
                os.close(fds[r])
                regions[r] = imp
                bases[r] = C.vmm_ptr(imp)
        heap = cls(rank, world, device, size, regions, bases)
        heap.local_bytes().zero_()
        if on_gpu:
            torch.cuda.synchronize(device)
        if world > 1:
            dist.barrier(group=group)
        return heap

    @classmethod
    def emulated(cls, world: int, size: int, device: int = 0) -> List["SymmetricHeap"]:
        """``world`` virtual ranks on one GPU (or on the CPU when the fake VMM backend is active)."""
        C = require_native()
        on_gpu = torch.cuda.is_available()
        if on_gpu:
            torch.cuda.set_device(device)
            torch.zeros(1, device=f"cuda:{device}")
            C.vmm_init(0)
        else:
            C.vmm_init(1)
        gran = C.vmm_granularity(device)
        size = _round_up(max(size, SIGNAL_BYTES + STATUS_BYTES + _ALIGN), gran)
        regions = [C.vmm_create(device, size, 0) for _ in range(world)]
        bases = [C.vmm_ptr(r) for r in regions]
        state = {"bump": SIGNAL_BYTES + STATUS_BYTES, "seq": {}, "slots": {}, "next_slot": 0}
        heaps = []
        for r in range(world):
            h = cls(r, world, device if on_gpu else -1, size, [regions[r]], bases, shared_state=state)
            h.local_bytes().zero_()
            heaps.append(h)
        if on_gpu:
            torch.cuda.synchronize(device)
        return heaps

    # ------------------------------------------------------------------ addressing
    def addr(self, offset: int = 0, rank: Optional[int] = None) -> int:
        return self.base[self.rank if rank is None else rank] + offset

    def peers(self, offset: int = 0) -> List[int]:
        """Address of byte ``offset`` in every rank's region (index = rank)."""
        return [b + offset for b in self.base]

    def tensor(self, offset: int, shape, dtype, rank: Optional[int] = None) -> torch.Tensor:
        """A tensor view of the region.  Views of a PEER region are for tests and host-side checks only:
        library kernels are never given peer memory as an operand."""
        return self.C.tensor_from_ptr(self.addr(offset, rank), list(shape), dtype, self.device)

    def local_bytes(self) -> torch.Tensor:
        return self.tensor(0, [self.size], torch.uint8)

    def alloc(self, nbytes: int, align: int = _ALIGN) -> int:
        """Bump allocation.  Collective by convention: every rank allocates the same sizes in the same order,
        so an offset means the same buffer on every rank."""
        st = self._state
        key = ("alloc_count", self.rank)
        n = st.get(key, 0)
        log = st.setdefault("alloc_log", [])
        if n < len(log):  # another virtual rank already performed this allocation: reuse its offset
            off, nb = log[n]
            assert nb == nbytes, "symmetric allocations must match across ranks"
        else:
            off = _round_up(st["bump"], align)
            if off + nbytes > self.size:
                raise MemoryError(f"symmetric heap exhausted: need {off + nbytes} of {self.size} bytes")
            st["bump"] = off + nbytes
            log.append((off, nbytes))
        st[key] = n + 1
        return off

    def alloc_tensor(self, shape, dtype) -> "SymTensor":
        n = 1
        for s in shape:
            n *= int(s)
        nbytes = n * torch.empty(0, dtype=dtype).element_size()
        off = self.alloc(max(nbytes, 16))
        return SymTensor(self, off, tuple(int(s) for s in shape), dtype)

    # ------------------------------------------------------------------ signals
    def signal_slots(self, name: str, count: int) -> int:
        """Reserve ``count`` consecutive uint32 words of the signal pad under ``name`` (same on every rank)."""
        st = self._state
        if name not in st["slots"]:
            if st["next_slot"] + count > SIGNAL_BYTES // 4:
                raise MemoryError("signal pad exhausted")
            st["slots"][name] = (st["next_slot"], count)
            st["next_slot"] += count
        return st["slots"][name][0]

    def sig_addr(self, slot: int, rank: Optional[int] = None) -> int:
        return self.addr(4 * slot, rank)

    def pads(self) -> List[int]:
        return self.peers(0)

    def signals(self, rank: Optional[int] = None) -> torch.Tensor:
        return self.tensor(0, [SIGNAL_BYTES // 4], torch.int32, rank)

    def next_seq(self, name: str) -> int:
        """Per-rank monotone sequence number for channel ``name``; every rank advances it in lock step."""
        key = (name, self.rank)
        v = self._state["seq"].get(key, 0) + 1
        self._state["seq"][key] = v
        return v

    def host_wait(self, slot: int, want: int, timeout_s: float = 120.0, poll_s: float = 0.0002) -> bool:
        """Poll one of this rank's signal words from the HOST until it reaches ``want`` (4-byte device->host copies on
        a private stream).  For waits that may last long (a decoder waiting for a prefill): no kernel spins on the GPU
        meanwhile.  Returns False on timeout."""
        import time as _time
        if self.device < 0:                        # host-memory heap (tests on the memfd backend): read the word itself
            word = self.tensor(4 * slot, [1], torch.int32)
            t0 = _time.monotonic()
            while ((int(word[0]) - want) & 0xFFFFFFFF) >= 0x80000000:
                if _time.monotonic() - t0 > timeout_s:
                    return False
                _time.sleep(poll_s)
            return True
        if not hasattr(self, "_poll_stream"):
            self._poll_stream = torch.cuda.Stream(device=self.device)
            self._poll_host = torch.zeros(1, dtype=torch.int32).pin_memory()
        word = self.tensor(4 * slot, [1], torch.int32)
        t0 = _time.monotonic()
        while True:
            with torch.cuda.stream(self._poll_stream):
                self._poll_host.copy_(word, non_blocking=True)
            self._poll_stream.synchronize()
            if ((int(self._poll_host[0]) - want) & 0xFFFFFFFF) < 0x80000000:
                return True
            if _time.monotonic() - t0 > timeout_s:
                return False
            _time.sleep(poll_s)

    # ------------------------------------------------------------------ status
    @property
    def status_addr(self) -> int:
        return self.addr(SIGNAL_BYTES)

    def status(self) -> torch.Tensor:
        return self.tensor(SIGNAL_BYTES, [8], torch.int32)

    def check_status(self, what: str = "kernel"):
        """Raise if a kernel recorded a timed-out wait or a bounds violation (reads 32 bytes back)."""
        st = self.status().cpu().tolist()
        if st[0] != 0:
            names = {1: "flag wait timed out", 2: "TMA full barrier timed out", 3: "smem stage never released",
                     4: "accumulator never ready", 5: "accumulator never released", 6: "index out of bounds"}
            self.status().zero_()
            raise RuntimeError(f"{what}: {names.get(st[0], 'error')} (code {st[0]}, where {st[1]}, cta {st[2]}, thread {st[3]})")

    # ------------------------------------------------------------------ teardown
    def close(self):
        if self._closed:
            return
        self._closed = True
        if self.device >= 0 and torch.cuda.is_available():
            torch.cuda.synchronize(self.device)
        for r in self._regions:
            if r is not None:
                self.C.vmm_destroy(r)
        self._regions = []


class SymTensor:
    """A buffer that exists at the same offset in every rank's region."""

    def __init__(self, heap: SymmetricHeap, offset: int, shape, dtype):
        self.heap, self.offset, self.shape, self.dtype = heap, offset, shape, dtype

    @property
    def local(self) -> torch.Tensor:
        return self.heap.tensor(self.offset, self.shape, self.dtype)

    def view_of(self, rank: int) -> torch.Tensor:
        return self.heap.tensor(self.offset, self.shape, self.dtype, rank)

    def addr(self, rank: Optional[int] = None) -> int:
        return self.heap.addr(self.offset, rank)

    def peers(self) -> List[int]:
        return self.heap.peers(self.offset)


# ---------------------------------------------------------------------------------------------------------
# fd exchange (SCM_RIGHTS over abstract-namespace Unix sockets)
# ---------------------------------------------------------------------------------------------------------
def _sock_name(token: str, rank: int) -> bytes:
    return b"\0fuselink-" + token.encode() + b"-" + str(rank).encode()


def _exchange_fds(token: str, rank: int, world: int, my_fd: int, barrier) -> List[int]:
    """Every rank receives one descriptor from every other rank.  Returns fds indexed by rank (own = -1)."""
    got: List[int] = [-1] * world
    srv = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
    srv.bind(_sock_name(token, rank))
    srv.listen(world)
    err: List[BaseException] = []

    def serve():
        try:
            for _ in range(world - 1):
                conn, _ = srv.accept()
                with conn:
                    msg, fds, _, _ = socket.recv_fds(conn, 16, 1)
                    got[int(msg.decode())] = fds[0]
        except BaseException as e:  # noqa: BLE001
            err.append(e)

    th = threading.Thread(target=serve, daemon=True)
    th.start()
    barrier()  # every listener is bound
    for peer in range(world):
        if peer == rank:
            continue
        c = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
        c.connect(_sock_name(token, peer))
        socket.send_fds(c, [str(rank).encode()], [my_fd])
        c.close()
    th.join(timeout=60)
    srv.close()
    if err:
        raise err[0]
    if th.is_alive() or any(got[r] < 0 for r in range(world) if r != rank):
        raise RuntimeError("file-descriptor exchange between ranks did not complete")
    return got
