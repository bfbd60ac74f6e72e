"""Python face of the path selector: monitor + selection policy + per-path statistics.

``PathSelector.plan(src, dst, nbytes)`` answers how one transfer is striped: always a direct stripe, plus relay
stripes over GPUs whose links the monitor reports idle, limited by the degree/step knobs of the reference's
bandwidth script (NCCL_FUSELINK_DEGREE / NCCL_FUSELINK_STEP, experiments/bw_test/run_bw_test.sbatch:37-38).
Behind one NVSwitch a single src->dst stream is bounded by the source's egress and the destination's ingress
whatever route it takes, so "direct" is a legitimate and frequent answer; relays pay off when a link is
degraded or marked dead, and the selector then routes around it.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Tuple

from .._ext import require_native
from ..utils.env import knobs
from ..utils.trace import TraceRecorder

TX, RX = 0, 1


@dataclass
class PathStats:
    status: int
    outstanding: int
    bandwidth_gbs: float


class PathSelector:
    def __init__(self, world: int, shm_name: str = "", own_table: bool = True, trace: Optional[TraceRecorder] = None):
        self.C = require_native()
        k = knobs()
        self.world = world
        self.degree, self.step = max(1, k.degree), max(1, k.step)
        self.min_stripe, self.align = k.min_stripe_bytes, k.chunk_bytes
        self.mon = self.C.monitor_open(shm_name, own_table, world, 1, k.monitor_timeout_us)
        self.owner = own_table
        if own_table:
            self.C.monitor_start(self.mon, max(10, k.monitor_timeout_us // 4))
        self.index = 0
        self.trace = trace
        self.direct_answers = 0
        self.relay_answers = 0

    def plan(self, src: int, dst: int, nbytes: int, allow_relay: bool = True) -> List[Tuple[int, int, int]]:
        now = self.C.monitor_now_ns()
        stripes = self.C.select_paths(self.mon, self.degree, self.step, self.min_stripe, self.align, allow_relay, src, dst, nbytes,
                                      self.index, now)
        self.index += 1
        self.C.monitor_post_bytes(self.mon, TX, src, nbytes, now)
        self.C.monitor_post_bytes(self.mon, RX, dst, nbytes, now)
        if len(stripes) > 1:
            self.relay_answers += 1
        else:
            self.direct_answers += 1
        if self.trace is not None:
            self.trace.instant("select", src=src, dst=dst, bytes=nbytes, paths=[p for p, _, _ in stripes])
        return stripes

    def complete(self, src: int, dst: int, nbytes: int, stripes: List[Tuple[int, int, int]]):
        now = self.C.monitor_now_ns()
        self.C.monitor_complete_bytes(self.mon, TX, src, nbytes, now)
        self.C.monitor_complete_bytes(self.mon, RX, dst, nbytes, now)
        for path, _, _ in stripes[1:]:
            self.C.monitor_release(self.mon, TX, path)

    def mark_dead(self, path: int, dead: bool = True):
        self.C.monitor_mark_dead(self.mon, TX, path, dead)
        self.C.monitor_mark_dead(self.mon, RX, path, dead)

    def stats(self) -> List[PathStats]:
        return [PathStats(self.C.monitor_status(self.mon, TX, p), self.C.monitor_outstanding(self.mon, TX, p),
                          self.C.monitor_bandwidth_gbs(self.mon, TX, p)) for p in range(self.world)]

    def close(self):
        if self.mon:
            self.C.monitor_close(self.mon, self.owner)
            self.mon = 0
