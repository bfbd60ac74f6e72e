"""bench.py on one GPU at a reduced size: the result line carries every key of the contract, the stock arm ran in the
same process, the end-to-end region declares its copies, and the other parts of the headline metric are there."""
import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_bench_line_on_one_gpu():
    cmd = [sys.executable, os.path.join(ROOT, "bench.py"), "--gpus", "1", "--steps", "3", "--warmup", "3", "--tokens", "1024",
           "--ffn", "2048", "--no-other"]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-3000:]
    lines = [l for l in out.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1, out.stdout[-2000:]
    r = json.loads(lines[0])
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling", "vs_baseline",
                "dtype", "data", "config", "clocks", "e2e", "gpu_launches", "roofline"):
        assert key in r, key
    assert r["n_gpus"] == 1 and r["steps"] == 3 and r["warmup"] == 3 and r["value"] > 0 and r["dtype"] == "bf16"
    assert r["gpu_launches"] >= 3 * 20, "every step launches this library's dispatch, GEMM and combine kernels"
    assert r["e2e"]["value"] > 0 and r["e2e"]["h2d_bytes_per_step"] == 1024 * 4096 * 2 and r["e2e"]["d2h_bytes_per_step"] == 4
    assert abs(r["e2e"]["last_loss"]) < 1e3
    base = r["vs_baseline"]
    assert base["value"] > 0 and base["ratio"] == pytest.approx(r["value"] / base["value"]) and base["expert_gemm"]
    assert r["roofline"]["hot_rank_rows"] == r["roofline"]["mean_rows"] == 1024 * 2
