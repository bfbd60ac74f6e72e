"""Metrics endpoint for the idleness monitor: the per-path table (state, outstanding bytes, smoothed bandwidth) in the
Prometheus text format, served over HTTP or printed once.

The reference's only structured state is the monitor's shared-memory table, readable by any process through
``getNICStatus`` (src/monitor.h:226-234).  This attaches to the same kind of table -- the one a ``fuselink-monitor``
daemon or a training process owns -- without taking part in path selection:

    python -m fuselink_b200.utils.metrics --shm /fuselink_monitor --paths 8 --port 9400     # serve /metrics
    python -m fuselink_b200.utils.metrics --shm /fuselink_monitor --paths 8 --once          # print and exit
"""
from __future__ import annotations

import argparse
import threading
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from typing import Optional

STATE_NAMES = {0: "idle", 1: "busy", 2: "borrowed", 3: "dead"}
DIRS = {0: "tx", 1: "rx"}


def render(C, mon: int, extra: Optional[dict] = None) -> str:
    """The monitor table ``mon`` (a handle from ``monitor_open``) as Prometheus exposition text."""
    n = C.monitor_num_paths(mon)
    lines = [
        "# HELP fuselink_path_state Path state (0 idle, 1 busy, 2 borrowed, 3 dead).",
        "# TYPE fuselink_path_state gauge",
    ]
    for d, dn in DIRS.items():
        for p in range(n):
            lines.append(f'fuselink_path_state{{dir="{dn}",path="{p}"}} {C.monitor_status(mon, d, p)}')
    lines += ["# HELP fuselink_path_outstanding_bytes Bytes posted on the path and not completed yet.",
              "# TYPE fuselink_path_outstanding_bytes gauge"]
    for d, dn in DIRS.items():
        for p in range(n):
            lines.append(f'fuselink_path_outstanding_bytes{{dir="{dn}",path="{p}"}} {C.monitor_outstanding(mon, d, p)}')
    lines += ["# HELP fuselink_path_bandwidth_gbs Exponentially smoothed completed bandwidth of the path in GB/s.",
              "# TYPE fuselink_path_bandwidth_gbs gauge"]
    for d, dn in DIRS.items():
        for p in range(n):
            lines.append(f'fuselink_path_bandwidth_gbs{{dir="{dn}",path="{p}"}} {C.monitor_bandwidth_gbs(mon, d, p):.6f}')
    lines += ["# HELP fuselink_borrow_decisions_total Paths handed out as relays since the table was created.",
              "# TYPE fuselink_borrow_decisions_total counter",
              f"fuselink_borrow_decisions_total {C.monitor_decisions(mon)}"]
    for k, v in (extra or {}).items():
        lines += [f"# TYPE fuselink_{k} gauge", f"fuselink_{k} {v}"]
    return "\n".join(lines) + "\n"


def plugin_counters(path: Optional[str] = None) -> dict:
    """Counters of the ncclNet plugin as loaded in THIS process (NCCL and ``ctypes`` share one copy of the library):
    selector decisions and fallbacks, stripes moved after a link failure, bytes stored through the same-host direct
    path, RDMA messages / pieces / work requests, memory registrations (made, answered from the cache, through a dma-buf).  Usable as ``extra`` of :func:`render` / :class:`MetricsServer`."""
    import ctypes
    import os
    if path is None:
        path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "lib", "libnccl-net-fuselink.so")
    lib = ctypes.CDLL(path)
    out = {}
    for name in ("decisions", "fallbacks", "failovers", "direct_bytes", "direct_msgs"):
        fn = getattr(lib, f"fuselink_plugin_{name}")
        fn.restype = ctypes.c_ulonglong
        out[f"plugin_{name}"] = int(fn())
    lib.fuselink_rdma_failovers.restype = ctypes.c_ulonglong
    out["plugin_rdma_failovers"] = int(lib.fuselink_rdma_failovers())
    m, p, w = ctypes.c_ulonglong(), ctypes.c_ulonglong(), ctypes.c_ulonglong()
    lib.fuselink_rdma_counters(ctypes.byref(m), ctypes.byref(p), ctypes.byref(w))
    out.update(plugin_rdma_messages=m.value, plugin_rdma_pieces=p.value, plugin_rdma_work_requests=w.value)
    r, h, d = ctypes.c_ulonglong(), ctypes.c_ulonglong(), ctypes.c_ulonglong()
    lib.fuselink_rdma_mr_counters(ctypes.byref(r), ctypes.byref(h), ctypes.byref(d))
    out.update(plugin_rdma_registrations=r.value, plugin_rdma_registration_cache_hits=h.value, plugin_rdma_dmabuf_registrations=d.value)
    return out


class MetricsServer:
    """``/metrics`` over HTTP on a background thread.  ``port=0`` picks a free port (see ``.port``)."""

    def __init__(self, C, mon: int, port: int = 9400, addr: str = "127.0.0.1", extra=None):
        outer = self

        class Handler(BaseHTTPRequestHandler):
            def do_GET(self):  # noqa: N802 - http.server's naming
                if self.path.rstrip("/") not in ("/metrics", ""):
                    self.send_error(404)
                    return
                body = render(outer.C, outer.mon, outer.extra() if callable(outer.extra) else outer.extra).encode()
                self.send_response(200)
                self.send_header("Content-Type", "text/plain; version=0.0.4")
                self.send_header("Content-Length", str(len(body)))
                self.end_headers()
                self.wfile.write(body)

            def log_message(self, *a):  # quiet
                pass

        self.C, self.mon, self.extra = C, mon, extra
        self.httpd = ThreadingHTTPServer((addr, port), Handler)
        self.port = self.httpd.server_address[1]
        self.thread = threading.Thread(target=self.httpd.serve_forever, daemon=True)
        self.thread.start()

    def close(self):
        self.httpd.shutdown()
        self.httpd.server_close()


def main():
    ap = argparse.ArgumentParser(prog="fuselink_b200.utils.metrics")
    ap.add_argument("--shm", required=True, help="name of the monitor's shared-memory table, e.g. /fuselink_monitor")
    ap.add_argument("--paths", type=int, default=8)
    ap.add_argument("--port", type=int, default=9400)
    ap.add_argument("--addr", default="127.0.0.1")
    ap.add_argument("--once", action="store_true")
    a = ap.parse_args()
    from .._ext import require_native
    from .env import Knobs
    C = require_native()
    mon = C.monitor_open(a.shm, False, a.paths, 1, Knobs().monitor_timeout_us)     # attach, never own
    if not mon:
        raise SystemExit(f"no monitor table named {a.shm}")
    if a.once:
        print(render(C, mon), end="")
        return
    srv = MetricsServer(C, mon, a.port, a.addr)
    print(f"serving http://{a.addr}:{srv.port}/metrics", flush=True)
    try:
        srv.thread.join()
    except KeyboardInterrupt:
        srv.close()


if __name__ == "__main__":
    main()
