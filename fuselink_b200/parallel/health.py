"""Host-side failure detection for multi-rank loops: heartbeats and clean departures through a key-value store.

The device kernels of this library wait on flags that peers write.  Such a wait is bounded (it gives up after its
limit and reports a status), but a rank that has died should be noticed on the HOST, before the next kernel that
would wait for it is launched.  Every rank publishes a heartbeat counter in a ``torch.distributed`` store from a
background thread; :meth:`Heartbeat.check` is called between steps and raises :class:`PeerLost` when a peer's counter
has stopped for longer than the timeout or when a peer announced that it is leaving.  Nothing here touches a GPU.

The reference has detection only at the verbs level (asynchronous port events, completion errors, QP retry limits:
src/plugin.cc:100-113, 1839-1861) and a lease rule in its monitor (a NIC not stamped for 160 us falls back to idle,
src/monitor.cpp:172-177); the heartbeat applies that lease idea to ranks.
"""
from __future__ import annotations

import threading
import time
from typing import Dict, List, Optional


class PeerLost(RuntimeError):
    def __init__(self, lost: List[int], left: List[int]):
        self.lost, self.left = lost, left
        super().__init__(f"ranks lost: {lost}; ranks that left: {left}")


class Heartbeat:
    """``store`` is any ``torch.distributed`` store every rank can reach (TCPStore, FileStore, the group's store).

    ``interval_s`` is the publishing period, ``timeout_s`` the age after which a silent peer counts as lost."""

    def __init__(self, store, rank: int, world: int, interval_s: float = 0.1, timeout_s: float = 1.0, prefix: str = "fl/hb"):
        self.store, self.rank, self.world = store, rank, world
        self.interval_s, self.timeout_s, self.prefix = interval_s, timeout_s, prefix
        self._stop = threading.Event()
        self._beat = 0
        self._seen: Dict[int, tuple] = {}          # rank -> (last counter value, local time it changed)
        self._publish()
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()

    def _key(self, kind: str, rank: int) -> str:
        return f"{self.prefix}/{kind}/{rank}"

    def _publish(self):
        self._beat += 1
        self.store.set(self._key("beat", self.rank), str(self._beat))

    def _run(self):
        while not self._stop.wait(self.interval_s):
            try:
                self._publish()
            except Exception:  # noqa: BLE001 - the store went away with the job
                return

    def _read(self, key: str) -> Optional[str]:
        try:
            if hasattr(self.store, "check") and not self.store.check([key]):
                return None
            return self.store.get(key).decode()
        except Exception:  # noqa: BLE001
            return None

    def status(self) -> Dict[int, str]:
        """rank -> "alive" | "left" | "lost" | "unknown" (never seen yet)."""
        now = time.monotonic()
        out = {}
        for r in range(self.world):
            if r == self.rank:
                out[r] = "alive"
                continue
            if self._read(self._key("left", r)) is not None:
                out[r] = "left"
                continue
            v = self._read(self._key("beat", r))
            if v is None:
                out[r] = "unknown"
                continue
            last = self._seen.get(r)
            if last is None or last[0] != v:
                self._seen[r] = (v, now)
                out[r] = "alive"
            else:
                out[r] = "alive" if now - last[1] <= self.timeout_s else "lost"
        return out

    def check(self) -> None:
        """Call between steps, with nothing of this rank in flight.  Raises PeerLost if a peer is gone."""
        st = self.status()
        lost = [r for r, s in st.items() if s == "lost"]
        left = [r for r, s in st.items() if s == "left"]
        if lost or left:
            raise PeerLost(lost, left)

    def survivors(self) -> List[int]:
        return [r for r, s in self.status().items() if s in ("alive", "unknown")]

    def wait_all_seen(self, timeout_s: float = 30.0) -> bool:
        """Block until every peer has published at least once (start-up rendezvous)."""
        t0 = time.monotonic()
        while time.monotonic() - t0 < timeout_s:
            if all(s != "unknown" for s in self.status().values()):
                return True
            time.sleep(self.interval_s / 2)
        return False

    def leave(self) -> None:
        """Announce a clean departure (between steps) and stop publishing."""
        self.store.set(self._key("left", self.rank), "1")
        self.close()

    def close(self) -> None:
        self._stop.set()
        self._thread.join(timeout=2 * self.interval_s + 1.0)


def renumber(survivors: List[int], rank: int) -> tuple:
    """(new rank, new world) of ``rank`` among the surviving ranks, in their old order: what a job needs to build a
    smaller process group and symmetric heap after a loss."""
    s = sorted(survivors)
    return s.index(rank), len(s)
