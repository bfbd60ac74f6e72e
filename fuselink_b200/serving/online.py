"""Trace-driven (online) disaggregated serving.

Reference behaviour (experiments/serving/online_main.cc:117-170, online_model.hh:41-98,447-491): a reader
thread replays a trace file whose lines look like ``ts: <seconds> prompt: <tokens> shared: <tokens> out: <tokens>``,
sleeping until each timestamp and queueing ``Request{timestamp, prompt_len, active_prompt_len = prompt - shared,
output_len}``; the context thread batches up to ``max_batch_size`` (20) queued requests, synthesises random
token ids, runs the prefill and sends a size header followed by the payload; the decode thread receives and
"decodes" (a 25 ms sleep per step in the reference).  It prints a communication-volume breakdown and the
send window.

Differences here: batches are variable-length (per-request block counts go through the KV kernel, so padding
is never transferred); two decode-side pools alternate so batch n+1 can land while batch n is decoded, with a
credit word from the decoder gating reuse; a request longer than ``input_len`` is rejected with a warning
instead of stalling the batcher forever (online_main.cc:144-145 spins on it).
"""
from __future__ import annotations

import queue
import re
import threading
import time
from dataclasses import dataclass
from typing import Callable, Iterable, List, Optional

import torch

from .disagg import HDR_INTS, HDR_LENS, HDR_OUTS, KVLink, ServeParams
from ..models.llama import LlamaShard
from ..utils.timing import device_sync, timing_event

MAX_BATCH = 20
_LINE = re.compile(r"ts:\s*([0-9.eE+-]+)\s+prompt:\s*(\d+)\s+shared:\s*(\d+)\s+out:\s*(\d+)")


@dataclass
class Request:
    timestamp: float
    prompt_len: int
    active_prompt_len: int
    output_len: int
    arrival: float = 0.0


def parse_trace(lines: Iterable[str]) -> List[Request]:
    out = []
    for ln in lines:
        m = _LINE.search(ln)
        if not m:
            continue
        ts, prompt, shared, outlen = float(m.group(1)), int(m.group(2)), int(m.group(3)), int(m.group(4))
        out.append(Request(ts, prompt, max(prompt - shared, 1), outlen))
    return out


class TraceReader(threading.Thread):
    """Replays the trace in (scaled) real time into a queue."""

    def __init__(self, requests: List[Request], q: "queue.Queue[Optional[Request]]", time_scale: float = 1.0):
        super().__init__(daemon=True)
        self.requests, self.q, self.scale = requests, q, time_scale

    def run(self):
        t0 = time.monotonic()
        for r in self.requests:
            delay = r.timestamp * self.scale - (time.monotonic() - t0)
            if delay > 0:
                time.sleep(delay)
            r.arrival = time.monotonic()
            self.q.put(r)
        self.q.put(None)


def next_batch(q: "queue.Queue[Optional[Request]]", max_batch: int, input_len: int, warn: Callable[[str], None] = print):
    """Block for one request, then take whatever else is queued, up to max_batch.  Returns (batch, finished)."""
    batch: List[Request] = []
    finished = False
    first = q.get()
    if first is None:
        return batch, True
    pending = [first]
    while pending or (len(batch) < max_batch and not q.empty()):
        r = pending.pop() if pending else q.get()
        if r is None:
            finished = True
            break
        if r.active_prompt_len > input_len:
            warn(f"request with {r.active_prompt_len} active prompt tokens exceeds input_len {input_len}: dropped")
            continue
        batch.append(r)
        if len(batch) >= max_batch:
            break
    return batch, finished


@dataclass
class BatchStats:
    batch: int
    prompt_tokens: int
    kv_bytes: int
    header_bytes: int
    send_ms: float
    prefill_ms: float


class OnlinePrefill:
    """Context side of the online experiment for one rank (TP shard)."""

    def __init__(self, p: ServeParams, model: LlamaShard, links: List[KVLink], dst_rank: int, seed: int = 0):
        self.p, self.model, self.links, self.dst = p, model, links, dst_rank
        m = p.model
        dev = model.embed.device
        self.dev = dev
        self.gen = torch.Generator(device=dev).manual_seed(seed)
        cb = p.context_blocks_per_req
        self.max_src_blocks = MAX_BATCH * cb
        n = self.max_src_blocks * m.layers * links[0].page_elems
        self.k_pool = torch.empty(n, dtype=p.dtype, device=dev)
        self.v_pool = torch.empty(n, dtype=p.dtype, device=dev)
        self.credit_slot = links[0].heap.signal_slots("online:credit", len(links))
        self.credit_pad = links[0].heap.alloc_tensor([16], torch.uint8)     # landing zone of the decoder's credit write
        self.batches = 0
        self.stats: List[BatchStats] = []

    def serve_batch(self, reqs: List[Request]) -> BatchStats:
        p, m = self.p, self.p.model
        B = len(reqs)
        assert 1 <= B <= MAX_BATCH and B <= p.batch_size
        bs = m.block_size
        lens = [r.active_prompt_len for r in reqs]
        S = (max(lens) + bs - 1) // bs * bs
        cb, mb = S // bs, p.max_blocks_per_req
        # the reference synthesises random token ids in [0, 31999] (online_main.cc:117-161)
        tokens = torch.randint(0, min(32000, m.vocab), (B, S), generator=self.gen, device=self.dev)
        src_bt = torch.arange(B * cb, dtype=torch.int32, device=self.dev).view(B, cb).contiguous()
        dst_bt = (torch.arange(B, dtype=torch.int32, device=self.dev).unsqueeze(1) * mb +
                  torch.arange(cb, dtype=torch.int32, device=self.dev).unsqueeze(0)).contiguous()
        nblocks = torch.tensor([(l + bs - 1) // bs for l in lens], dtype=torch.int32, device=self.dev)
        link = self.links[self.batches % len(self.links)]
        use = self.batches // len(self.links)
        heap = link.heap
        C = link.C
        e0, e1, e2 = (timing_event(self.dev) for _ in range(3))
        e0.record()
        # prefill computes on the padded batch; the last real position of each request gives its first token
        last_pos = torch.tensor([l - 1 for l in lens], dtype=torch.long, device=self.dev)
        first = self.model.prefill(tokens, self.k_pool, self.v_pool, src_bt, None, last_pos=last_pos)
        e1.record()
        if use > 0:   # wait until the decoder has released this pool (credit = number of batches it finished on it)
            self._wait_credit(use)
        link.seq += 1
        hdr = torch.zeros(HDR_INTS, dtype=torch.int64, device=self.dev)
        hdr[0], hdr[1], hdr[2], hdr[3] = B, S, mb, self.batches
        hdr[4:4 + B] = first
        hdr[HDR_LENS:HDR_LENS + B] = torch.tensor(lens, dtype=torch.int64, device=self.dev)
        hdr[HDR_OUTS:HDR_OUTS + B] = torch.tensor([r.output_len for r in reqs], dtype=torch.int64, device=self.dev)
        link.send_layers(self.dst, self.k_pool, self.v_pool, B * cb, src_bt, dst_bt, nblocks, 0, m.layers)
        link.send_layers(self.dst, self.k_pool, self.v_pool, B * cb, src_bt, dst_bt, torch.zeros_like(nblocks), 0, 1, hdr=hdr,
                         final=True, num_ctas=1)
        e2.record()
        device_sync(self.dev)
        kv_bytes = int(nblocks.sum().item()) * m.layers * link.page_elems * 2 * p.elem_bytes
        st = BatchStats(B, sum(lens), kv_bytes, HDR_INTS * 8, e1.elapsed_time(e2), e0.elapsed_time(e1))
        self.stats.append(st)
        self.batches += 1
        return st


    def _wait_credit(self, use: int):
        """The long part of the wait is a host poll (a decoder may work on the pool for seconds); the device wait
        behind it only orders the following kernels after the credit."""
        heap = self.links[0].heap
        slot = self.credit_slot + self.batches % len(self.links)
        if not heap.host_wait(slot, use, 600.0):
            raise TimeoutError(f"decoder did not release pool {self.batches % len(self.links)} within 600 s")
        self.links[0].C.wait_flags([(heap.sig_addr(slot), use)], heap.status_addr)

    def send_end(self):
        """Tell the decoder that the trace is over: a header with batch size 0 on the next pool."""
        link = self.links[self.batches % len(self.links)]
        use = self.batches // len(self.links)
        if use > 0:
            self._wait_credit(use)
        link.seq += 1
        hdr = torch.zeros(HDR_INTS, dtype=torch.int64, device=self.dev)
        hdr[3] = self.batches
        one = torch.zeros(1, 1, dtype=torch.int32, device=self.dev)
        link.send_layers(self.dst, self.k_pool, self.v_pool, 1, one, one, torch.zeros(1, dtype=torch.int32, device=self.dev), 0, 1,
                         hdr=hdr, final=True, num_ctas=1)
        device_sync(self.dev)
        self.batches += 1


class OnlineDecode:
    """Decode side: waits for a batch, generates `steps` tokens per request (or sleeps `sleep_ms` per step like the
    reference's stand-in), then returns the pool to the sender through the credit word."""

    def __init__(self, p: ServeParams, model: Optional[LlamaShard], links: List[KVLink], src_rank: int, sleep_ms: float = 0.0):
        self.p, self.model, self.links, self.src, self.sleep_ms = p, model, links, src_rank, sleep_ms
        self.credit_slot = links[0].heap.signal_slots("online:credit", len(links))
        self.credit_pad = links[0].heap.alloc_tensor([16], torch.uint8)
        self.batches = 0
        self.done_on = [0] * len(links)

    def serve_batch(self, max_steps: int) -> dict:
        p = self.p
        i = self.batches % len(self.links)
        link = self.links[i]
        heap = link.heap
        link.seq += 1
        link.wait_final()
        device_sync(link.k_pool.local.device)
        heap.check_status("online decode wait")
        hdr = link.hdr.local.cpu()
        B, S, mb = int(hdr[0]), int(hdr[1]), int(hdr[2])
        if B == 0:                                   # end of the trace (OnlinePrefill.send_end)
            self.batches += 1
            return {"batch": 0, "padded_len": 0, "steps": 0, "generated": None, "output_lens": []}
        lens = hdr[HDR_LENS:HDR_LENS + B].clone()
        outs = hdr[HDR_OUTS:HDR_OUTS + B].clone()
        dev = link.k_pool.local.device
        tokens = hdr[4:4 + B].to(dev)
        pos = lens.to(dev)
        bt = (torch.arange(B, dtype=torch.int32, device=dev).unsqueeze(1) * mb + torch.arange(mb, dtype=torch.int32, device=dev).unsqueeze(0)).contiguous()
        steps = min(max_steps, p.num_decoding_step)
        gen = [tokens]
        for _ in range(steps):
            if self.model is None or self.sleep_ms > 0:
                time.sleep(self.sleep_ms / 1e3)
            else:
                tokens = self.model.decode_step(tokens, pos, link.k_pool.local, link.v_pool.local, bt, link.pool_blocks)
                pos = pos + 1
                gen.append(tokens)
        device_sync(dev)
        # give the pool back: credit word on the SENDER's pad counts batches finished on this pool
        self.done_on[i] += 1
        link.C.put_chunks([(self.credit_pad.addr(), self.credit_pad.addr(self.src), 16,
                            heap.sig_addr(self.credit_slot + i, self.src), 2, 0)], 16, 0, False, 1, 32, heap.status_addr)
        self.batches += 1
        return {"batch": B, "padded_len": S, "steps": steps, "generated": torch.stack(gen, 1), "output_lens": outs.tolist()}
