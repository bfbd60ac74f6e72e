"""Disaggregated serving: a prefill (context) stage and a decode stage on different GPUs, linked by the fused
KV hand-off kernel.

Reference behaviour (experiments/serving/main.cc:184-202, model.hh:253-337,420-529): ranks below world/2 run
the context stage, the rest decode; after the WHOLE prefill the context rank sends first tokens, the whole K
pool, the whole V pool, the block table and the block counts to rank + world/2 in one NCCL group, and the
decoder then generates tokens.  It prints elapsed time, KV send time and their ratio (main.cc:228-239).

Here the pairing (rank -> rank + world/2) and the reports are kept; the transfer is `kv_pack_send`: only the
pages in use move, they are re-laid-out for the decode pool on the fly, the small messages ride along as one
header, and each layer's pages leave as soon as that layer has been computed (a side stream ordered by events),
so the transfer overlaps the rest of the prefill.

``KVLink`` is the transfer object, ``PrefillStage`` / ``DecodeStage`` wrap the model, ``run_offline`` is the
two-stage experiment; all of them also work with both stages as virtual ranks on ONE GPU (emulated heap).
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Optional

import torch

from .._ext import require_native
from ..models.llama import KV_BLHSD, KV_LBSHD, LlamaConfig, LlamaShard
from ..parallel.symm import SymmetricHeap
from ..utils.timing import device_sync, timing_event

HDR_MAX_BATCH = 32
HDR_TOKENS, HDR_LENS, HDR_OUTS = 4, 4 + HDR_MAX_BATCH, 4 + 2 * HDR_MAX_BATCH
HDR_INTS = 4 + 3 * HDR_MAX_BATCH   # [batch, prompt_len, max_blocks, batch_index] + first tokens + prompt lengths + output lengths


@dataclass
class ServeParams:
    """The experiment's knobs (TestParams of the reference, experiments/serving/model.hh:31-49)."""
    model: LlamaConfig
    batch_size: int = 16
    input_len: int = 2048
    num_decoding_step: int = 256
    tp_size: int = 1
    dtype: torch.dtype = torch.bfloat16     # --precision of the reference's binaries (fp16 / fp32 there); KV pools use it too

    @property
    def elem_bytes(self) -> int:
        return torch.empty((), dtype=self.dtype).element_size()

    @property
    def kv_dim_units(self) -> int:
        """Head dimension as the KV kernel sees it: the kernel moves 2-byte elements, so a 4-byte type is a head twice
        as wide (the innermost run of a page is one head vector either way)."""
        return self.model.head_dim * self.elem_bytes // 2

    @property
    def block_size(self) -> int:
        return self.model.block_size

    @property
    def max_blocks_per_req(self) -> int:          # ceil((input + decode) / block), model.hh:100-103
        return (self.input_len + self.num_decoding_step + self.block_size - 1) // self.block_size

    @property
    def context_blocks_per_req(self) -> int:
        return (self.input_len + self.block_size - 1) // self.block_size


class KVLink:
    """Decode-side pools inside the symmetric heap + the flags and header of the hand-off.  Collective: both
    stages construct it with the same arguments so that offsets agree."""

    def __init__(self, heap: SymmetricHeap, p: ServeParams, kv_heads_local: int, name: str = "kv"):
        self.heap, self.p, self.kvh = heap, p, kv_heads_local
        m = p.model
        self.pool_blocks = p.batch_size * p.max_blocks_per_req
        self.page_elems = kv_heads_local * m.block_size * m.head_dim
        n = self.pool_blocks * m.layers * self.page_elems
        self.k_pool = heap.alloc_tensor([n], p.dtype)
        self.v_pool = heap.alloc_tensor([n], p.dtype)
        self.hdr = heap.alloc_tensor([HDR_INTS], torch.int64)
        self.layer_flags = heap.signal_slots(f"{name}:layers", m.layers)
        self.final_flag = heap.signal_slots(f"{name}:final", 1)
        self.seq = 0
        self.C = require_native()
        dev = self.k_pool.local.device
        self.cta_counter = torch.zeros(1, dtype=torch.int32, device=dev)

    # ---- prefill side -------------------------------------------------------------------------------------
    def send_layers(self, dst_rank: int, src_k, src_v, src_blocks: int, src_bt, dst_bt, nblocks, l0: int, l1: int,
                    hdr: Optional[torch.Tensor] = None, final: bool = False, num_ctas: int = 0):
        m = self.p.model
        flag = self.heap.sig_addr(self.final_flag if final else self.layer_flags + l0, dst_rank)
        self.C.kv_pack_send(src_k, src_v, self.k_pool.addr(dst_rank), self.v_pool.addr(dst_rank), KV_BLHSD, KV_LBSHD,
                            src_blocks, self.pool_blocks, m.layers, self.kvh, m.block_size, self.p.kv_dim_units, l0, l1, src_bt, dst_bt,
                            nblocks, hdr, self.hdr.addr(dst_rank) if hdr is not None else 0, flag, self.seq, self.cta_counter,
                            num_ctas, self.heap.status_addr)

    # ---- decode side --------------------------------------------------------------------------------------
    def wait_final(self, host_timeout_s: float = 300.0):
        """Wait for the header + all pages of hand-off number ``seq``.  The long part of the wait is a host poll (the
        prefill may take seconds); the device wait that follows only orders later kernels after the flag."""
        if not self.heap.host_wait(self.final_flag, self.seq, host_timeout_s):
            raise TimeoutError(f"KV hand-off {self.seq} did not arrive within {host_timeout_s} s")
        self.C.wait_flags([(self.heap.sig_addr(self.final_flag), self.seq)], self.heap.status_addr)

    def wait_layer(self, l: int):
        self.C.wait_flags([(self.heap.sig_addr(self.layer_flags + l), self.seq)], self.heap.status_addr)


@dataclass
class StageReport:
    role: str
    elapsed_ms: float = 0.0
    compute_ms: float = 0.0
    kv_ms: float = 0.0              # device time of the KV hand-off kernels (prefill) / of the wait (decode)
    kv_bytes: int = 0
    tokens: int = 0
    extra: dict = field(default_factory=dict)


class PrefillStage:
    def __init__(self, p: ServeParams, model: LlamaShard, link: KVLink, dst_rank: int, pipeline_layers: bool = True):
        self.p, self.model, self.link, self.dst = p, model, link, dst_rank
        self.pipeline = pipeline_layers
        m = p.model
        dev = model.embed.device
        self.ctx_blocks = p.batch_size * p.context_blocks_per_req
        n = self.ctx_blocks * m.layers * link.page_elems
        self.k_pool = torch.empty(n, dtype=p.dtype, device=dev)
        self.v_pool = torch.empty(n, dtype=p.dtype, device=dev)
        B, cb, mb = p.batch_size, p.context_blocks_per_req, p.max_blocks_per_req
        # source pages: request-major; destination pages: the decode pool reserves max_blocks_per_req per request
        self.src_bt = torch.arange(B * cb, dtype=torch.int32, device=dev).view(B, cb).contiguous()
        self.dst_bt = (torch.arange(B, dtype=torch.int32, device=dev).unsqueeze(1) * mb +
                       torch.arange(cb, dtype=torch.int32, device=dev).unsqueeze(0)).contiguous()
        self.nblocks = torch.full((B,), cb, dtype=torch.int32, device=dev)
        # the KV hand-off runs on a side stream beside the prefill; on host tensors (tests that model the kernels) in line
        self.side = torch.cuda.Stream(device=dev) if dev.type == "cuda" else None
        self.dev = dev
        self.hdr = torch.zeros(HDR_INTS, dtype=torch.int64, device=dev)

    def run(self, tokens: torch.Tensor) -> StageReport:
        p, link = self.p, self.link
        link.seq += 1
        cuda = self.side is not None
        main = torch.cuda.current_stream() if cuda else None
        e0, e1, k0, k1 = (timing_event(self.dev) for _ in range(4))
        first_kv = [True]

        def after_main():
            """The side stream continues from what the main stream has enqueued so far."""
            if cuda:
                ev = torch.cuda.Event()
                ev.record(main)
                self.side.wait_event(ev)

        def on_layer(l: int):
            if not self.pipeline:
                return
            with torch.cuda.stream(self.side):
                after_main()
                if first_kv[0]:
                    k0.record(self.side)
                    first_kv[0] = False
                link.send_layers(self.dst, self.k_pool, self.v_pool, self.ctx_blocks, self.src_bt, self.dst_bt, self.nblocks, l, l + 1)

        e0.record(main)
        first = self.model.prefill(tokens, self.k_pool, self.v_pool, self.src_bt, on_layer)
        e1.record(main)
        self.hdr[0], self.hdr[1], self.hdr[2] = p.batch_size, p.input_len, p.max_blocks_per_req
        self.hdr[4:4 + p.batch_size] = first
        with torch.cuda.stream(self.side):
            after_main()
            if not self.pipeline:
                k0.record(self.side)
                link.send_layers(self.dst, self.k_pool, self.v_pool, self.ctx_blocks, self.src_bt, self.dst_bt, self.nblocks, 0,
                                 p.model.layers)
            # header + final flag: a zero-layer-cost launch that only copies the control block
            link.send_layers(self.dst, self.k_pool, self.v_pool, self.ctx_blocks, self.src_bt, self.dst_bt,
                             torch.zeros_like(self.nblocks), 0, 1, hdr=self.hdr, final=True, num_ctas=1)
            k1.record(self.side)
        if cuda:
            main.wait_stream(self.side)
        device_sync(self.dev)
        kv_bytes = 2 * self.ctx_blocks * p.model.layers * link.page_elems * p.elem_bytes
        return StageReport("prefill", elapsed_ms=e0.elapsed_time(k1), compute_ms=e0.elapsed_time(e1), kv_ms=k0.elapsed_time(k1),
                           kv_bytes=kv_bytes, tokens=p.batch_size * p.input_len)


class DecodeStage:
    """Greedy decoding over the paged pool.  The per-token step is launch-bound (hundreds of small kernels), so it
    is captured once in a CUDA graph and replayed; ``use_graph=False`` keeps the eager loop."""

    def __init__(self, p: ServeParams, model: LlamaShard, link: KVLink, use_graph: bool = True):
        self.p, self.model, self.link = p, model, link
        dev = model.embed.device
        B, mb = p.batch_size, p.max_blocks_per_req
        self.bt = (torch.arange(B, dtype=torch.int32, device=dev).unsqueeze(1) * mb +
                   torch.arange(mb, dtype=torch.int32, device=dev).unsqueeze(0)).contiguous()
        self.dev = dev
        self.use_graph = use_graph and dev.type == "cuda"
        self.graph = None
        self.g_tokens = torch.zeros(B, dtype=torch.long, device=dev)
        self.g_pos = torch.zeros(B, dtype=torch.long, device=dev)
        self.g_out = None

    def _step(self, tokens, pos):
        link = self.link
        return self.model.decode_step(tokens, pos, link.k_pool.local, link.v_pool.local, self.bt, link.pool_blocks)

    def _capture(self):
        """Capture one decode step on static buffers.  The step writes K/V at g_pos, so the capture (which runs the
        step for real during warm-up) is done at a scratch position that the first real step overwrites anyway."""
        try:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for _ in range(2):
                    self._step(self.g_tokens, self.g_pos)
            torch.cuda.current_stream().wait_stream(side)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self.g_out = self._step(self.g_tokens, self.g_pos)
            self.graph = g
        except Exception as e:  # noqa: BLE001 - capture is an optimisation; the eager loop is always valid
            self.graph = None
            self.use_graph = False
            print(f"[fuselink] decode graph capture failed ({type(e).__name__}: {e}); running eagerly")

    def decode(self, tokens: torch.Tensor):
        """Generate num_decoding_step tokens after `tokens` ([B] first tokens).  Returns (generated [B, 1+steps],
        device ms of the loop)."""
        p = self.p
        d0, d1 = timing_event(self.dev), timing_event(self.dev)
        out = [tokens]
        pos = torch.full((p.batch_size,), p.input_len, dtype=torch.long, device=tokens.device)
        if self.use_graph and self.graph is None:
            self.g_tokens.copy_(tokens)
            self.g_pos.copy_(pos)
            self._capture()                     # one-off set-up, outside the timed loop
        d0.record()
        for _ in range(p.num_decoding_step):
            if self.graph is not None:
                self.g_tokens.copy_(tokens)
                self.g_pos.copy_(pos)
                self.graph.replay()
                tokens = self.g_out.clone()
            else:
                tokens = self._step(tokens, pos)
            out.append(tokens)
            pos = pos + 1
        d1.record()
        device_sync(self.dev)
        return torch.stack(out, 1), d0.elapsed_time(d1)

    def run(self) -> StageReport:
        p, link = self.p, self.link
        link.seq += 1
        w0, w1 = timing_event(self.dev), timing_event(self.dev)
        w0.record()
        link.wait_final()                       # header + every layer's pages have landed
        w1.record()
        tokens = link.hdr.local[4:4 + p.batch_size].clone()
        device_sync(self.dev)
        t_first = time.monotonic()              # first token is on the decode side: time-to-first-token ends here
        gen, ms = self.decode(tokens)
        rep = StageReport("decode", elapsed_ms=w0.elapsed_time(w1) + ms, compute_ms=ms, kv_ms=w0.elapsed_time(w1),
                          tokens=p.batch_size * p.num_decoding_step)
        rep.extra["t_first_token"] = t_first
        rep.extra["generated"] = gen
        rep.extra["graph"] = self.graph is not None
        return rep


def make_prompts(p: ServeParams, device, seed: int = 0) -> torch.Tensor:
    g = torch.Generator(device=device).manual_seed(seed)
    return torch.randint(0, p.model.vocab, (p.batch_size, p.input_len), generator=g, device=device)
