"""Arithmetic helpers: roofline model of the MoE step, env knobs, chunking policy of the copy kernels, trace recorder."""
import json
import os

import pytest


def test_moe_step_model_counts_three_gemms_forward_and_twice_that_backward():
    from fuselink_b200.utils import roofline as rl
    T, H, F, k = 8192, 4096, 14336, 2
    m = rl.moe_step_model(T, 1, H, F, k, T * k)
    per_row_fwd = 2 * H * 2 * F + 2 * F * H                      # gate|up GEMM + down GEMM
    assert m["flops"] == T * k * 3 * per_row_fwd                 # forward + dgrad + wgrad
    assert abs(m["flops"] / (T * k) / 1e6 - 3 * 352.3) < 1.0     # "352 MFLOP per routed token" per pass
    assert m["nvlink_bytes"] == 0                                # one GPU: nothing crosses NVLink
    m8 = rl.moe_step_model(T, 8, H, F, k, 3 * T * k)
    assert m8["nvlink_bytes"] == 3 * T * k * H * 2 * 4 * 7 / 8
    p = rl.peaks()
    assert m8["target_ms"] == pytest.approx(max(m8["flops"] / (p.bf16_tflops_sustained * 1e12), m8["nvlink_bytes"] / 770e9) * 1e3)
    assert rl.gemm_fraction(p.bf16_tflops * 1e12, 1000.0) == pytest.approx(1.0)
    assert rl.hbm_fraction(p.hbm_gbs * 1e9, 1000.0) == pytest.approx(1.0)


def test_peaks_come_from_the_measured_file_when_present(tmp_path, monkeypatch):
    from fuselink_b200.utils import roofline as rl
    monkeypatch.setattr(rl, "_ROOT", str(tmp_path))
    assert rl.peaks().source == "fallback" and rl.peaks().bf16_tflops == 1590.0
    (tmp_path / "MEASURED_PEAKS.json").write_text(json.dumps({"hbm_gbs": 6500.0, "bf16_tflops": 1600.0, "bf16_tflops_sustained": 1390.0}))
    p = rl.peaks()
    assert (p.source, p.hbm_gbs, p.bf16_tflops_sustained) == ("measured", 6500.0, 1390.0)


def test_env_knobs_follow_the_reference_names(monkeypatch):
    from fuselink_b200.utils.env import Knobs
    monkeypatch.setenv("NCCL_FUSELINK_DEGREE", "3")
    monkeypatch.setenv("NCCL_FUSELINK_STEP", "2")
    monkeypatch.setenv("NCCL_FUSELINK_PRIORITY_DEV", "5")
    k = Knobs()
    assert (k.degree, k.step, k.priority_dev) == (3, 2, 5)
    assert k.monitor_timeout_us == 160 and k.steps_in_flight == 8            # MONITOR_TIMEOUT_US, FUSELINK_STEPS of the reference


def test_chunking_policy_of_the_copy_kernels():
    from fuselink_b200.ops.comm import chunking
    for nbytes in (1, 1000, 16 << 10, (3 << 20) + 48, 1 << 30):
        chunk, n = chunking(nbytes)
        assert chunk % 16 == 0 and chunk > 0                     # 16-byte vectors / bulk copies
        assert (n - 1) * chunk < nbytes <= n * chunk
    chunk, n = chunking(1 << 30)
    assert chunk >= 64 << 10                                     # large messages: at least 64 KiB per remote flag update


def test_trace_recorder_writes_chrome_trace(tmp_path):
    from fuselink_b200.utils.trace import TraceRecorder
    tr = TraceRecorder()
    with tr.span("step", n=1):
        tr.instant("decision", path=3)
        tr.counter("outstanding", tx=7)
    out = tmp_path / "t.json"
    tr.dump(str(out))
    ev = json.load(open(out))["traceEvents"]
    assert {e["ph"] for e in ev} == {"X", "i", "C"}
    assert [e for e in ev if e["ph"] == "X"][0]["dur"] >= 0


def test_bench_reference_arm_reports_why_it_is_unavailable():
    """`bench.py --impl reference` must print one JSON line with "impl": "reference" and exit 0 even without a GPU."""
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "1"],
                         capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and isinstance(line["unavailable"], str) and "\n" not in line["unavailable"]


def test_every_environment_variable_read_by_the_sources_is_documented():
    """docs/environment.md lists every FUSELINK_* / NCCL_* / FL_* name that appears as a string in the package, the benches
    and the experiment scripts."""
    import os
    import re
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    doc = open(os.path.join(root, "docs", "environment.md")).read()
    documented = set(re.findall(r"`((?:FUSELINK|NCCL|FL)_[A-Z0-9_]+)`", doc))
    names = set()
    tops = [os.path.join(root, d) for d in ("fuselink_b200", "bench", "experiments")] + [os.path.join(root, "bench.py")]
    for top in tops:
        files = [top] if os.path.isfile(top) else [os.path.join(d, f) for d, _, fs in os.walk(top) for f in fs]
        for path in files:
            if not path.endswith((".py", ".cc", ".cu", ".cpp", ".h", ".cuh", ".sh")):
                continue
            text = open(path, errors="replace").read()
            names |= set(re.findall(r"\"((?:FUSELINK|NCCL|FL)_[A-Z0-9_]+)\"", text))
            if path.endswith(".sh"):
                names |= set(re.findall(r"\b((?:FUSELINK|NCCL)_[A-Z0-9_]+)=", text))
    names = {n for n in names if not n.startswith(("NCCL_PTR_", "NCCL_LOG_", "NCCL_NET_HANDLE", "NCCL_NET_MAX", "NCCL_ALL", "NCCL_INIT", "NCCL_NET_DEVICE"))}
    missing = sorted(names - documented)
    assert not missing, f"not in docs/environment.md: {missing}"


def test_bench_result_line_is_printed_once_even_when_the_run_stalls():
    """bench.py's ResultLine: a second emit prints nothing; an armed timer prints the line with an error in place of the
    end-to-end part and ends the process with status 0 while the main thread is stuck."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    code = ("import sys, time; sys.path.insert(0, %r); import bench\n"
            "parts = {}\n"
            "r = bench.ResultLine(0, lambda p: {'value': 1.5, 'e2e': p.get('e2e'), 'roofline': p.get('roofline')}, parts)\n"
            "mode = sys.argv[1]\n"
            "if mode == 'twice':\n"
            "    r.arm(30.0); r.disarm(); parts['e2e'] = {'value': 2}; parts['roofline'] = {'x': 1}; r.emit(); parts['e2e'] = {'value': 3}; r.emit()\n"
            "else:\n"
            "    r.arm(0.3); time.sleep(20); print('never')\n") % root
    twice = subprocess.run([sys.executable, "-c", code, "twice"], capture_output=True, text=True, timeout=60)
    assert twice.returncode == 0 and twice.stdout.strip() == '{"value": 1.5, "e2e": {"value": 2}, "roofline": {"x": 1}}'
    import time
    t0 = time.time()
    stuck = subprocess.run([sys.executable, "-c", code, "stuck"], capture_output=True, text=True, timeout=60)
    assert stuck.returncode == 0 and time.time() - t0 < 10 and "never" not in stuck.stdout
    import json
    line = json.loads(stuck.stdout.strip())
    assert line["value"] == 1.5 and "did not finish" in line["e2e"]["error"] and line["roofline"] is None
