"""Point-to-point, striped-relay and all-to-all transfers over the symmetric heap.

All transfers are one launch of the chunked put kernel (csrc/kernels/comm_kernels.cu) on the sender plus,
where the receiver has to know, one launch of the flag-wait kernel on the receiver.  Nothing here calls
NCCL; NCCL is what these are benchmarked against (bench/p2p_sweep.py, bench/a2a_sweep.py).

Completion accounting uses monotone arrival counters: the sender adds 1 per chunk to a word in the
receiver's signal pad, both sides derive the number of chunks from the byte count with ``chunking()``, and
the receiver waits for its running total.  No word is ever reset.
"""
from __future__ import annotations

from typing import Optional, Sequence, Tuple

import torch

from .._ext import require_native
from ..parallel.symm import SymmetricHeap, SymTensor
from ..utils.env import knobs

FLAG_NONE, FLAG_SEQ_PER_CHUNK, FLAG_COUNT = 0, 1, 2
_NUM_SMS = 148


def chunking(nbytes: int, chunk_bytes: Optional[int] = None) -> Tuple[int, int]:
    """(chunk_bytes, number_of_chunks) both sides of a transfer agree on.

    Large messages use the configured chunk (512 KiB, the reference's NCCL_P2P_NET_CHUNKSIZE setting); smaller
    ones are cut so that every SM gets about one chunk, never below 64 KiB.
    """
    cfg = chunk_bytes or _chunk_default()
    if nbytes <= 0:
        return cfg, 0
    c = cfg
    # about one chunk per SM for mid sizes; a chunk is never cut below 64 KiB (a CTA streams it through a ring of
    # 16 KiB slots, and every chunk costs one remote flag update)
    while c > _chunk_min() and nbytes // c < _NUM_SMS:
        c //= 2
    c = max(16, (c + 15) // 16 * 16)
    return c, (nbytes + c - 1) // c


_CHUNK_DEFAULT = None
_CHUNK_MIN = None


def _chunk_min() -> int:
    global _CHUNK_MIN
    if _CHUNK_MIN is None:
        _CHUNK_MIN = max(16, knobs().chunk_min_bytes)
    return _CHUNK_MIN



def _chunk_default() -> int:
    global _CHUNK_DEFAULT
    if _CHUNK_DEFAULT is None:
        _CHUNK_DEFAULT = knobs().chunk_bytes
    return _CHUNK_DEFAULT


_COPY_CTAS = None


def _launch_shape(total_chunks: int, engine: str) -> Tuple[int, int]:
    global _COPY_CTAS
    if _COPY_CTAS is None:
        _COPY_CTAS = knobs().copy_ctas
    if engine == "bulk":
        return _COPY_CTAS or min(max(total_chunks, 1), 3 * _NUM_SMS), 32
    return _COPY_CTAS or min(max(total_chunks, 1), 2 * _NUM_SMS), 512


class Channel:
    """A set of arrival counters (one per source rank) plus the running totals both sides keep."""

    def __init__(self, heap: SymmetricHeap, name: str, engine: Optional[str] = None):
        self.heap, self.name = heap, name
        self.C = require_native()
        self.slot0 = heap.signal_slots(f"chan:{name}", heap.world)
        self.expected = [0] * heap.world
        self.engine = engine or knobs().copy_engine
        self.counters = None      # optional pinned int64[world]: bytes this rank has finished sending to each peer

    def attach_counters(self, selector) -> torch.Tensor:
        """Let the put kernel report completed bytes per destination straight to the monitor: a pinned host array the
        kernel adds to (system-scope atomics) and the monitor's sweeper thread reads (`fl_monitor_attach_counters`)."""
        self.counters = torch.zeros(max(self.heap.world, 64), dtype=torch.int64).pin_memory()
        self.C.monitor_attach_counters(selector.mon, 0, self.counters.data_ptr())
        # device words in which a launch adds up its finished bytes, so that it touches the host counter once (see FlPutArgs)
        dev = self.heap.status().device
        self.counter_scratch = torch.zeros(16, dtype=torch.int64, device=dev) if dev.type == "cuda" else None
        return self.counters

    # -- sender ------------------------------------------------------------------------------------
    def put(self, src: torch.Tensor, dst_rank: int, dst_offset: int, nbytes: Optional[int] = None,
            chunk_bytes: Optional[int] = None) -> int:
        """Copy ``nbytes`` of the local tensor ``src`` to byte ``dst_offset`` of rank ``dst_rank``'s region and
        bump that rank's arrival counter for this source.  Returns the number of chunks signalled."""
        nbytes = src.numel() * src.element_size() if nbytes is None else nbytes
        cb, n = chunking(nbytes, chunk_bytes)
        if n == 0:
            return 0
        seg = (src.data_ptr(), self.heap.addr(dst_offset, dst_rank), nbytes,
               self.heap.sig_addr(self.slot0 + self.heap.rank, dst_rank), FLAG_COUNT, 0)
        ctas, threads = _launch_shape(n, self.engine)
        ctr = [self.counters.data_ptr() + 8 * dst_rank] if self.counters is not None else []
        scratch = self.counter_scratch.data_ptr() if ctr and getattr(self, "counter_scratch", None) is not None else 0
        self.C.put_chunks([seg], cb, 0, self.engine == "bulk", ctas, threads, self.heap.status_addr, ctr, scratch)
        return n

    def put_many(self, items: Sequence[Tuple[int, int, int, int]], chunk_bytes: int) -> None:
        """items: (src_addr, dst_rank, dst_offset, nbytes); one launch, at most 8 items."""
        segs = []
        total = 0
        for src_addr, dst_rank, dst_off, nbytes in items:
            if nbytes <= 0:
                continue
            segs.append((src_addr, self.heap.addr(dst_off, dst_rank), nbytes,
                         self.heap.sig_addr(self.slot0 + self.heap.rank, dst_rank), FLAG_COUNT, 0))
            total += (nbytes + chunk_bytes - 1) // chunk_bytes
        if not segs:
            return
        ctas, threads = _launch_shape(total, self.engine)
        self.C.put_chunks(segs, chunk_bytes, 0, self.engine == "bulk", ctas, threads, self.heap.status_addr)

    # -- receiver ----------------------------------------------------------------------------------
    def expect(self, src_rank: int, nbytes: int, chunk_bytes: Optional[int] = None) -> None:
        _, n = chunking(nbytes, chunk_bytes)
        self.expected[src_rank] += n

    def expect_chunks(self, src_rank: int, n: int) -> None:
        self.expected[src_rank] += n

    def wait(self, src_ranks: Optional[Sequence[int]] = None) -> None:
        """Enqueue a wait (on the current stream) until everything announced with expect() has arrived."""
        ranks = range(self.heap.world) if src_ranks is None else src_ranks
        flags = [(self.heap.sig_addr(self.slot0 + r), self.expected[r] & 0xFFFFFFFF) for r in ranks if self.expected[r] > 0]
        for i in range(0, len(flags), 16):
            self.C.wait_flags(flags[i:i + 16], self.heap.status_addr)


def barrier(heap: SymmetricHeap, name: str = "barrier", signal: bool = True, wait: bool = True) -> None:
    """Device-side barrier over all ranks of the heap (one tiny kernel on the current stream)."""
    C = require_native()
    slot0 = heap.signal_slots(f"bar:{name}", heap.world)
    if signal:
        heap._state.setdefault("barseq", {})
        key = (name, heap.rank)
        heap._state["barseq"][key] = heap._state["barseq"].get(key, 0) + 1
    seq = heap._state.get("barseq", {}).get((name, heap.rank), 0)
    C.barrier(heap.pads(), slot0, heap.rank, heap.world, seq, signal, wait, heap.status_addr)


def all_to_all(chan: Channel, send: torch.Tensor, recv: SymTensor, wait: bool = True) -> None:
    """Uniform all-to-all: ``send`` is [world, n] on this rank, block p goes to rank p's ``recv[rank]``.

    One launch pushes all blocks (segment p -> peer p); with ``wait`` the call also enqueues the wait for the
    blocks of every other rank.
    """
    heap = chan.heap
    W = heap.world
    assert send.shape[0] == W and send.is_contiguous()
    per = send[0].numel() * send.element_size()
    cb, n = chunking(per)
    for r in range(W):
        chan.expected[r] += n
    ctas, threads = _launch_shape(n * W, chan.engine)
    want = [e & 0xFFFFFFFF for e in chan.expected] if wait else []
    chan.C.all_to_all(send.data_ptr(), recv.peers(), per, heap.rank, heap.pads(), chan.slot0, cb, want,
                      chan.engine == "bulk", ctas, threads, heap.status_addr)


def all_to_all_v(chan: Channel, send: torch.Tensor, send_offsets: Sequence[int], send_bytes: Sequence[int],
                 recv: SymTensor, dst_offsets: Sequence[int], recv_bytes: Sequence[int], wait: bool = True) -> None:
    """Variable all-to-all in bytes.  ``dst_offsets[p]`` is where this rank's block lands inside rank p's ``recv``;
    ``recv_bytes[r]`` is what rank r sends here (both known from a prior size exchange)."""
    heap = chan.heap
    cb = knobs().chunk_bytes
    base = send.data_ptr()
    items = [(base + send_offsets[p], p, recv.offset + dst_offsets[p], send_bytes[p]) for p in range(heap.world)]
    chan.put_many(items, cb)
    for r in range(heap.world):
        chan.expect_chunks(r, (recv_bytes[r] + cb - 1) // cb)
    if wait:
        chan.wait()


class StripedP2P:
    """One logical src -> dst transfer striped over the direct path and idle relay GPUs.

    Collective over the heap: every rank calls ``transfer`` with the same arguments; the source pushes each
    stripe (stripe 0 straight to the destination, stripe i into relay i's staging buffer, one flag per
    chunk), each relay forwards its stripe chunk by chunk as the flags appear, the destination waits for its
    arrival counter.  This is the reference's multi-path idea (a channel's buffer lives on a relay GPU,
    src/plugin.cc:1201, src/fuselink.cc:43-56) with explicit stripes instead of per-channel VA remaps.

    Flow control: a relay's staging buffer has two halves used in turn (per relay: its k-th stripe goes to half
    k % 2), and a relay counts the stripes it has finished forwarding in a word of its own signal pad.  Before a
    source writes a relay's k-th stripe it waits (on its stream, reading the relay's word over NVLink) until the
    relay has forwarded its first k - 1 stripes, i.e. until the half it is about to overwrite has been drained.
    Transfers may therefore be issued back to back; a stripe must fit in half the staging buffer.
    """

    def __init__(self, heap: SymmetricHeap, name: str, staging_bytes: int, engine: Optional[str] = None):
        self.heap = heap
        self.C = require_native()
        self.engine = engine or knobs().copy_engine
        self.chunk = knobs().chunk_bytes
        self.half_chunks = max(1, staging_bytes // 2 // self.chunk)
        self.half_bytes = self.half_chunks * self.chunk
        self.staging = heap.alloc_tensor([2 * self.half_bytes], torch.uint8)
        self.chunk_flags = heap.signal_slots(f"relay:{name}:chunks", 2 * self.half_chunks)
        self.arrive = heap.signal_slots(f"relay:{name}:arrive", 1)
        self.forwarded = heap.signal_slots(f"relay:{name}:forwarded", 1)      # on the relay: stripes it has passed on
        self.token = heap.alloc_tensor([32], torch.uint8)                     # 16 B payload + 16 B landing place of the count bump
        self.seq = 0
        self.arrived_expected = 0
        self.relayed = [0] * heap.world                                       # stripes given to each relay so far (same on every rank)

    def transfer(self, src_rank: int, dst_rank: int, src: Optional[torch.Tensor], dst: SymTensor, nbytes: int,
                 stripes: Sequence[Tuple[int, int, int]]) -> None:
        """stripes: (path, offset, bytes) as produced by the selector; path == dst_rank is the direct stripe."""
        heap = self.heap
        self.seq += 1
        cb = self.chunk
        me = heap.rank
        total_chunks = sum((b + cb - 1) // cb for _, _, b in stripes if b > 0)
        relays = [(path, off, b) for path, off, b in stripes if b > 0 and path != dst_rank]
        assert len({p for p, _, _ in relays}) == len(relays), "one stripe per relay and transfer"
        halves = {path: self.relayed[path] % 2 for path, _, _ in relays}
        if me == src_rank:
            segs, credits = [], []
            for path, off, b in stripes:
                if b <= 0:
                    continue
                if path == dst_rank:
                    segs.append((src.data_ptr() + off, dst.addr(dst_rank) + off, b,
                                 heap.sig_addr(self.arrive, dst_rank), FLAG_COUNT, 0))
                else:
                    assert b <= self.half_bytes, "stripe larger than half the relay staging buffer"
                    h = halves[path]
                    if self.relayed[path] >= 2:       # the stripe that last used this half has left the relay
                        credits.append((heap.sig_addr(self.forwarded, path), (self.relayed[path] - 1) & 0xFFFFFFFF))
                    segs.append((src.data_ptr() + off, self.staging.addr(path) + h * self.half_bytes, b,
                                 heap.sig_addr(self.chunk_flags + h * self.half_chunks, path), FLAG_SEQ_PER_CHUNK, 0))
            if credits:
                self.C.wait_flags(credits, heap.status_addr)
            ctas, threads = _launch_shape(total_chunks, self.engine)
            self.C.put_chunks(segs, cb, self.seq, self.engine == "bulk", ctas, threads, heap.status_addr)
        for path, off, b in relays:
            if path == me and me != src_rank:
                h = halves[path]
                seg = (self.staging.addr() + h * self.half_bytes, dst.addr(dst_rank) + off, b, heap.sig_addr(self.arrive, dst_rank),
                       FLAG_COUNT, heap.sig_addr(self.chunk_flags + h * self.half_chunks))
                n = (b + cb - 1) // cb
                ctas, threads = _launch_shape(n, self.engine)
                self.C.put_chunks([seg], cb, self.seq, self.engine == "bulk", ctas, threads, heap.status_addr)
                # stream-ordered after the forward: one more stripe has left this relay (a 16-byte local put whose
                # arrival count is the word the source waits on)
                bump = (self.token.addr(), self.token.addr() + 16, 16, heap.sig_addr(self.forwarded), FLAG_COUNT, 0)
                self.C.put_chunks([bump], 16, 0, False, 1, 32, heap.status_addr)
        for path, _, _ in relays:
            self.relayed[path] += 1
        if me == dst_rank:
            self.arrived_expected += total_chunks
            self.C.wait_flags([(heap.sig_addr(self.arrive), self.arrived_expected & 0xFFFFFFFF)], heap.status_addr)
