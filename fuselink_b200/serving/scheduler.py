"""Batch scheduler of the context stage of online serving.

The reference's context thread takes whatever is queued, first come first served, up to its maximum batch of 20
(experiments/serving/online_main.cc:117-161), and leaves a file for a scheduler empty (experiments/serving/scheduler.h).
This module is that scheduler: it drains the arrival queue into a waiting list and forms the next batch from it under a
policy, with two limits -- requests per batch and active prompt tokens per batch (the prefill cost, hence the time to first
token of everyone in the batch, grows with the tokens, not with the requests).

    fcfs     arrival order (the reference's behaviour when the token limit is off)
    sjf      fewest active prompt tokens first: short prompts are not held up behind long ones
    aged     sjf on ``tokens - aging * waited_seconds``: a long prompt moves forward as it waits, so it cannot starve

A request whose active prompt is longer than the model's input length is dropped with a warning instead of being retried
forever (the reference's loop spins on it, online_main.cc:144-145).
"""
from __future__ import annotations

import queue
import time
from typing import Callable, List, Optional, Tuple

from .online import Request

POLICIES = ("fcfs", "sjf", "aged")


class Scheduler:
    def __init__(self, q: "queue.Queue[Optional[Request]]", max_batch: int, input_len: int, policy: str = "fcfs",
                 max_batch_tokens: int = 0, aging_tokens_per_s: float = 1000.0, warn: Callable[[str], None] = print,
                 clock: Callable[[], float] = time.monotonic):
        assert policy in POLICIES and max_batch >= 1
        self.q, self.max_batch, self.input_len, self.policy = q, max_batch, input_len, policy
        self.max_batch_tokens, self.aging, self.warn, self.clock = max_batch_tokens, aging_tokens_per_s, warn, clock
        self.waiting: List[Request] = []
        self.closed = False                 # the end-of-trace marker has been seen
        self.dropped = 0

    def _admit(self, r: Optional[Request]) -> None:
        if r is None:
            self.closed = True
        elif r.active_prompt_len > self.input_len:
            self.dropped += 1
            self.warn(f"request with {r.active_prompt_len} active prompt tokens exceeds input_len {self.input_len}: dropped")
        else:
            if not r.arrival:
                r.arrival = self.clock()
            self.waiting.append(r)

    def _drain(self, block: bool) -> None:
        if block and not self.waiting and not self.closed:
            self._admit(self.q.get())
        while not self.closed:
            try:
                self._admit(self.q.get_nowait())
            except queue.Empty:
                break

    def _order(self) -> List[Request]:
        if self.policy == "fcfs":
            return list(self.waiting)
        now = self.clock()
        key = (lambda r: r.active_prompt_len) if self.policy == "sjf" else \
              (lambda r: r.active_prompt_len - self.aging * (now - r.arrival))
        return sorted(self.waiting, key=key)             # stable: ties keep arrival order

    def next_batch(self) -> Tuple[List[Request], bool]:
        """Blocks until at least one request waits (or the trace has ended).  Returns (batch, finished); finished means the
        trace has ended and nothing waits any more."""
        while True:
            self._drain(block=True)
            if self.waiting or self.closed:
                break
        batch: List[Request] = []
        tokens = 0
        for r in self._order():
            if len(batch) >= self.max_batch:
                break
            if self.max_batch_tokens and batch and tokens + r.active_prompt_len > self.max_batch_tokens:
                if self.policy == "fcfs":
                    break                                # arrival order is kept: nothing overtakes the request that did not fit
                continue
            batch.append(r)
            tokens += r.active_prompt_len
        taken = set(map(id, batch))
        self.waiting = [r for r in self.waiting if id(r) not in taken]
        return batch, self.closed and not self.waiting
