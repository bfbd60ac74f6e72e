"""Device timing helpers: CUDA-event section timers (the reference's CudaTimer, experiments/serving/model.hh:51-89)
and a max-over-ranks reduction for anything multi-GPU."""
from __future__ import annotations

from contextlib import contextmanager
from typing import Dict, List

import torch


class _HostEvent:
    """Stand-in with the two methods of a CUDA timing event that the serving code uses, on the host clock."""

    def record(self, stream=None):
        import time
        self.t = time.perf_counter()

    def elapsed_time(self, other: "_HostEvent") -> float:
        return (other.t - self.t) * 1e3


def timing_event(device):
    """A CUDA timing event for a CUDA device; on the CPU (tests that model the kernels) the host clock."""
    return torch.cuda.Event(enable_timing=True) if torch.device(device).type == "cuda" else _HostEvent()


def device_sync(device) -> None:
    if torch.device(device).type == "cuda":
        torch.cuda.synchronize()


class CudaTimer:
    """Named sections timed with CUDA events on the current stream; totals are read after a synchronize."""

    def __init__(self):
        self._open: Dict[str, torch.cuda.Event] = {}
        self._pairs: Dict[str, List[tuple]] = {}

    def start(self, name: str):
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        self._open[name] = ev

    def stop(self, name: str):
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        self._pairs.setdefault(name, []).append((self._open.pop(name), ev))

    @contextmanager
    def section(self, name: str):
        self.start(name)
        try:
            yield
        finally:
            self.stop(name)

    def totals_ms(self) -> Dict[str, float]:
        torch.cuda.synchronize()
        return {k: sum(a.elapsed_time(b) for a, b in v) for k, v in self._pairs.items()}

    def report(self) -> str:
        t = self.totals_ms()
        return "  ".join(f"{k}: {v:.3f} ms" for k, v in t.items())


def max_over_ranks(ms: float, device=None) -> float:
    """Slowest rank's time (what a multi-GPU number must be quoted as)."""
    import torch.distributed as dist

    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return ms
    t = torch.tensor([ms], dtype=torch.float64, device=device or torch.cuda.current_device())
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def time_kernel(fn, warmup: int = 3, iters: int = 10, flush_l2: bool = True) -> float:
    """Mean device time of ``fn`` in ms.  Between iterations a buffer larger than the 126 MB L2 is rewritten so
    that every iteration starts cold."""
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda") if flush_l2 else None
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        if flush is not None:
            flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        total += e0.elapsed_time(e1)
    return total / iters
