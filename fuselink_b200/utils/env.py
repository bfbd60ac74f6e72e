"""Environment knobs.

The names are the ones the reference reads (``NCCL_PARAM`` macro, src/extern/param.h:19-28; list in
src/plugin.cc:87-117,584,887,1410 and experiments/bw_test/run_bw_test.sbatch:34-46) plus the ones this
framework adds (prefix ``FUSELINK_``).  The native plugin reads the same variables in C++
(csrc/net/params.cc); this module is the Python view used by the torch-side selector and benches.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field


def _int(name: str, default: int) -> int:
    v = os.environ.get(name)
    if v is None or v == "":
        return default
    try:
        return int(v, 0)
    except ValueError:
        return default


@dataclass
class Knobs:
    # reference knobs
    priority_dev: int = field(default_factory=lambda: _int("NCCL_FUSELINK_PRIORITY_DEV", 0))
    degree: int = field(default_factory=lambda: _int("NCCL_FUSELINK_DEGREE", 1))
    step: int = field(default_factory=lambda: _int("NCCL_FUSELINK_STEP", 1))
    chunk_bytes: int = field(default_factory=lambda: _int("NCCL_P2P_NET_CHUNKSIZE", 512 * 1024))
    buff_size: int = field(default_factory=lambda: _int("NCCL_BUFFSIZE", 4 * 1024 * 1024))
    nchannels_per_peer: int = field(default_factory=lambda: _int("NCCL_NCHANNELS_PER_NET_PEER", 4))
    # framework knobs
    monitor_timeout_us: int = field(default_factory=lambda: _int("FUSELINK_MONITOR_TIMEOUT_US", 160))
    min_stripe_bytes: int = field(default_factory=lambda: _int("FUSELINK_MIN_STRIPE_BYTES", 4 * 1024 * 1024))
    copy_engine: str = field(default_factory=lambda: os.environ.get("FUSELINK_COPY_ENGINE", "bulk"))  # bulk | ldst
    copy_ctas: int = field(default_factory=lambda: _int("FUSELINK_COPY_CTAS", 0))
    chunk_min_bytes: int = field(default_factory=lambda: _int("FUSELINK_CHUNK_MIN", 64 * 1024))   # mid sizes are cut into about one chunk per SM, never below this
    steps_in_flight: int = 8  # FUSELINK_STEPS in the reference (src/fuselink.h:14)


def knobs() -> Knobs:
    return Knobs()
