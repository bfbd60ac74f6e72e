"""Chrome-trace (chrome://tracing / Perfetto JSON) recorder for host-side events: selector decisions, transfers,
step phases.  Optional NVTX ranges are emitted when torch.cuda.nvtx is usable."""
from __future__ import annotations

import json
import os
import threading
import time
from contextlib import contextmanager
from typing import List


class TraceRecorder:
    def __init__(self, nvtx: bool = False):
        self.events: List[dict] = []
        self.lock = threading.Lock()
        self.nvtx = nvtx
        self.t0 = time.perf_counter_ns()

    def _ts(self) -> float:
        return (time.perf_counter_ns() - self.t0) / 1e3

    def instant(self, name: str, **args):
        with self.lock:
            self.events.append({"name": name, "ph": "i", "ts": self._ts(), "pid": os.getpid(), "tid": threading.get_ident() % 100000, "s": "t", "args": args})

    @contextmanager
    def span(self, name: str, **args):
        start = self._ts()
        if self.nvtx:
            import torch
            torch.cuda.nvtx.range_push(name)
        try:
            yield
        finally:
            if self.nvtx:
                import torch
                torch.cuda.nvtx.range_pop()
            with self.lock:
                self.events.append({"name": name, "ph": "X", "ts": start, "dur": self._ts() - start, "pid": os.getpid(),
                                    "tid": threading.get_ident() % 100000, "args": args})

    def counter(self, name: str, **values):
        with self.lock:
            self.events.append({"name": name, "ph": "C", "ts": self._ts(), "pid": os.getpid(), "args": values})

    def dump(self, path: str):
        with self.lock, open(path, "w") as f:
            json.dump({"traceEvents": self.events, "displayTimeUnit": "ms"}, f)
