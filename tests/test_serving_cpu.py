"""Host-side logic of the serving experiments without a GPU: trace parsing and replay, batching rules of the online
experiment, paged-attention geometry of the reference's TestModel, KV sizes per precision, command-line surface."""
import queue
import subprocess
import sys
import time

import torch

from fuselink_b200.models.llama import MODEL_ZOO
from fuselink_b200.serving.disagg import ServeParams
from fuselink_b200.serving.online import MAX_BATCH, Request, TraceReader, next_batch, parse_trace


def test_trace_lines_are_parsed_like_the_reference_reader():
    """`ts: .. prompt: .. shared: .. out: ..` -> Request{timestamp, prompt_len, active = prompt - shared, output}
    (experiments/serving/online_model.hh:41-98); other lines are skipped."""
    reqs = parse_trace(["# comment", "ts: 0.5 prompt: 1000 shared: 200 out: 30", "garbage", "ts: 1.25e0 prompt: 64 shared: 64 out: 1"])
    assert [(r.timestamp, r.prompt_len, r.active_prompt_len, r.output_len) for r in reqs] == [(0.5, 1000, 800, 30), (1.25, 64, 1, 1)]


def test_batching_takes_what_is_queued_up_to_the_limit_and_drops_oversized_requests():
    q = queue.Queue()
    for i in range(MAX_BATCH + 5):
        q.put(Request(0.0, 100 + i, 100 + i, 4))
    warned = []
    batch, finished = next_batch(q, MAX_BATCH, 4096, warned.append)
    assert len(batch) == MAX_BATCH and not finished                      # "max batch = 20" of the reference
    q.put(Request(0.0, 9000, 9000, 4))                                   # longer than input_len: the reference spins on it forever
    q.put(None)
    batch, finished = next_batch(q, MAX_BATCH, 4096, warned.append)
    assert len(batch) == 5 and finished and len(warned) == 1 and "exceeds input_len" in warned[0]
    q.put(None)
    assert next_batch(q, MAX_BATCH, 4096) == ([], True)


def test_trace_reader_replays_in_scaled_real_time():
    reqs = parse_trace([f"ts: {0.05 * i} prompt: 10 shared: 0 out: 1" for i in range(5)])
    q = queue.Queue()
    t0 = time.monotonic()
    TraceReader(reqs, q, time_scale=1.0).start()
    got = []
    while True:
        r = q.get(timeout=5)
        if r is None:
            break
        got.append(r.arrival - t0)
    assert len(got) == 5
    assert all(b >= a for a, b in zip(got, got[1:])) and 0.15 < got[-1] < 1.0


def test_paged_attention_geometry_and_kv_sizes():
    """max_num_block_per_req = ceil((input + decode) / block) (experiments/serving/model.hh:100-103); KV bytes per
    request follow the element size of the chosen precision."""
    m = MODEL_ZOO["opt_13b"]
    p = ServeParams(m, batch_size=15, input_len=2048, num_decoding_step=100)
    assert p.block_size == m.block_size
    assert p.context_blocks_per_req == -(-2048 // m.block_size)
    assert p.max_blocks_per_req == -(-(2048 + 100) // m.block_size)
    assert (p.elem_bytes, p.kv_dim_units) == (2, m.head_dim)
    p32 = ServeParams(m, dtype=torch.float32)
    assert (p32.elem_bytes, p32.kv_dim_units) == (4, 2 * m.head_dim)
    # the reference's example: opt_13b, 15 x 2048 tokens -> 2 (K,V) x 40 layers x 40 heads x 128 x 2 B x 30720 tokens ~ 25 GB
    kv = 2 * m.layers * m.kv_heads * m.head_dim * p.elem_bytes * 15 * 2048
    assert abs(kv / 1e9 - 25.2) < 0.2


def test_command_line_has_the_reference_flags():
    out = subprocess.run([sys.executable, "-m", "fuselink_b200.serving", "--help"], capture_output=True, text=True, timeout=120)
    assert out.returncode == 0
    for flag in ("--model_name", "--model_path", "--vocab_json_path", "--precision", "--input_len", "--batch_size", "--block_size",
                 "--num_decoding_step", "--tp_size", "--tracepath"):
        assert flag in out.stdout, flag
    bad = subprocess.run([sys.executable, "-m", "fuselink_b200.serving", "--model_name", "no_such_model"], capture_output=True, text=True, timeout=120)
    assert bad.returncode != 0 and "unknown model" in bad.stderr


def test_model_benchmark_script_runs_prefill_and_decode_on_one_group():
    """experiments/run_model_benchmark.sh (the reference's benchmark_tp2 / benchmark_tp4 jobs): tensor parallelism 2 over gloo."""
    import json
    import os
    import subprocess
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, DEVICE="cpu", MODEL="tiny_opt", INPUT_LEN="64", TP="2", DECODE_STEPS="3", BATCH="2", PORT="29673")
    out = subprocess.run([os.path.join(root, "experiments", "run_model_benchmark.sh")], env=env, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr[-3000:]
    row = json.loads([l for l in out.stdout.splitlines() if l.startswith("{")][-1])
    assert row["tp"] == 2 and row["decode_steps"] == 3 and row["prefill_ms"] > 0 and row["decode_ms_per_token"] > 0


def test_trace_generator_writes_what_the_reader_parses():
    from fuselink_b200.serving.online import parse_trace
    from fuselink_b200.serving.tracegen import generate
    lines = generate(requests=200, rate=50.0, prompt_min=16, prompt_max=512, shared_fraction=0.5, out_min=2, out_max=9, seed=4)
    assert lines == generate(requests=200, rate=50.0, prompt_min=16, prompt_max=512, shared_fraction=0.5, out_min=2, out_max=9, seed=4)
    reqs = parse_trace(lines)
    assert len(reqs) == 200
    ts = [r.timestamp for r in reqs]
    assert ts == sorted(ts) and 2.0 < ts[-1] < 8.0                       # 200 arrivals at 50 per second: about 4 s
    assert all(16 <= r.prompt_len <= 512 and 2 <= r.output_len <= 9 for r in reqs)
    assert all(r.prompt_len - r.prompt_len // 2 <= r.active_prompt_len <= r.prompt_len for r in reqs)


def _sched(policy, reqs, **kw):
    import queue
    from fuselink_b200.serving.online import Request
    from fuselink_b200.serving.scheduler import Scheduler
    q = queue.Queue()
    for i, (tokens, arrival) in enumerate(reqs):
        q.put(Request(timestamp=float(i), prompt_len=tokens, active_prompt_len=tokens, output_len=4, arrival=arrival))
    q.put(None)
    warnings = []
    s = Scheduler(q, policy=policy, warn=warnings.append, clock=lambda: 100.0, **kw)
    batches = []
    while True:
        b, done = s.next_batch()
        if b:
            batches.append([r.active_prompt_len for r in b])
        if done:
            return batches, warnings, s


def test_scheduler_policies_and_limits():
    reqs = [(900, 99.0), (50, 99.1), (400, 99.2), (60, 99.3), (5000, 99.4), (70, 99.5)]
    # the reference's behaviour: arrival order, up to the batch limit; the oversized request is dropped, not retried forever
    b, w, s = _sched("fcfs", reqs, max_batch=3, input_len=1024)
    assert b == [[900, 50, 400], [60, 70]] and len(w) == 1 and s.dropped == 1
    # token limit in arrival order: a batch closes where the next request does not fit, nothing overtakes
    b, _, _ = _sched("fcfs", reqs, max_batch=20, input_len=1024, max_batch_tokens=1000)
    assert b == [[900, 50], [400, 60, 70]]
    # shortest first, with the same limit: short prompts go together, the long one alone
    b, _, _ = _sched("sjf", reqs, max_batch=20, input_len=1024, max_batch_tokens=1000)
    assert b == [[50, 60, 70, 400], [900]]
    # a single request over the token limit still runs (alone) instead of waiting forever
    b, _, _ = _sched("sjf", [(800, 99.0)], max_batch=4, input_len=1024, max_batch_tokens=100)
    assert b == [[800]]


def test_aged_policy_lets_a_long_prompt_overtake_once_it_has_waited():
    # 900 tokens, waiting 2 s at 400 tokens per second of ageing -> counts as 100: ahead of the fresh 300-token request
    b, _, _ = _sched("aged", [(900, 98.0), (300, 100.0), (50, 100.0)], max_batch=2, input_len=1024, aging_tokens_per_s=400.0)
    assert b == [[50, 900], [300]]
    b, _, _ = _sched("sjf", [(900, 98.0), (300, 100.0), (50, 100.0)], max_batch=2, input_len=1024)
    assert b == [[50, 300], [900]]
