"""The Python side of the fused paths run on the CPU: the device entry points are replaced by the functional model of
tests/cpu_kernel_model.py and the symmetric heap lives in host memory.  First the MoE step (ops/moe.py: buffers, slices,
parities, phases, fp8 arm, shadow experts) with the ranks emulated in one process -- the scenario and the checks are the
GPU test's own, against the same fp32 oracle -- then MoE, DLRM, striped transfers and a training loop between REAL
processes that share the heap, where barriers and waits are real."""
import pytest
import torch

from fuselink_b200 import have_native

pytestmark = pytest.mark.skipif(not have_native() or torch.cuda.is_available(), reason="CPU-only run of the kernel model")


def _run_on_model(*args, **kw):
    import cpu_kernel_model
    from test_moe_gpu import _run
    with cpu_kernel_model.installed():
        _run(*args, device="cpu", T=64, H=128, Fd=256, **kw)


@pytest.mark.parametrize("world", [1, 2, 4])
def test_moe_forward_backward_on_the_model(world):
    _run_on_model(world)


def test_two_steps_with_the_update_fused_into_wgrad():
    _run_on_model(2, sgd=0.05, steps=2)


@pytest.mark.parametrize("world", [1, 2])
def test_fp8_arm_on_the_model(world):
    """Quantise -> fp8 GEMM -> quantise ... in forward and dgrad, wgrad in bf16: what is quantised when, with which scales,
    and that the forward's quantised weights serve the transposed use in backward."""
    _run_on_model(world, fp8=True)


def test_fp8_arm_with_shadow_experts_on_the_model():
    _run_on_model(2, fp8=True, shadow=(0,))


@pytest.mark.parametrize("world,shadow", [(2, (0,)), (4, (0, 5)), (1, (2,)), (4, (7, 1, 2))])
def test_shadow_experts_on_the_model(world, shadow):
    """Rows of a shadowed expert stay on their rank; outputs, input gradients and the summed weight gradients equal the oracle's."""
    _run_on_model(world, shadow=shadow)


def test_shadow_experts_two_steps_fused_update_keeps_the_copies_identical():
    _run_on_model(2, sgd=0.05, steps=2, shadow=(1,))


@pytest.mark.parametrize("world,shadow,spread", [
    (2, (0,), [[0.5, 0.5], [0.25, 0.75]]),
    (4, (0, 5), [[1, 0, 0, 0], [0.2, 0.3, 0.5, 0], [0, 0, 0.4, 0.6], [0.25, 0.25, 0.25, 0.25]]),
    (2, (4, -1), [[0.0, 1.0], [1.0, 0.0]]),
])
def test_shadow_rows_spread_over_the_copies_on_the_model(world, shadow, spread):
    """A shadowed expert's rows computed by other ranks' copies: outputs, input gradients and summed weight gradients as before."""
    _run_on_model(world, shadow=shadow, spread=spread)
    _run_on_model(world, shadow=shadow, spread=spread, sgd=0.05, steps=2)


def test_shadowed_rows_do_not_cross_ranks():
    """With every expert shadowed nothing is sent: each rank's counters show exactly its own tokens."""
    import cpu_kernel_model
    from fuselink_b200.models.moe import MoELayer
    from fuselink_b200.ops import moe as M
    from fuselink_b200.parallel.symm import SymmetricHeap
    E, W, T, k = 4, 2, 32, 2
    cfg = M.MoEConfig(hidden=128, ffn=256, num_experts=E, topk=k, tokens=T)
    heaps = SymmetricHeap.emulated(W, 32 << 20)
    try:
        with cpu_kernel_model.installed():
            layers = [MoELayer(cfg, heaps[r], r, W, device="cpu", seed=2, name="s", shadow_experts=list(range(E))) for r in range(W)]
            xs = [torch.randn(T, 128).to(torch.bfloat16) for _ in range(W)]
            routes = [l.route(x) for l, x in zip(layers, xs)]
            for r in range(W):
                M.moe_forward_dispatch(layers[r].ws, xs[r], routes[r][1].contiguous())
            for r in range(W):
                c = layers[r].ws.counts_now()
                assert int(c[:E // W].sum()) == 0 and int(c[E // W:].sum()) == T * k
    finally:
        for h in heaps:
            h.close()


def test_shadowing_the_hot_experts_levels_the_load():
    """8 ranks, one expert each, Zipf(1.2) router bias: the busiest rank's row count (what sets the step time) falls from
    about a third of all rows to well under twice the mean when the three hottest experts are shadowed."""
    import cpu_kernel_model
    from fuselink_b200.models.moe import MoELayer
    from fuselink_b200.ops import moe as M
    from fuselink_b200.parallel.symm import SymmetricHeap
    E = W = 8
    T, k = 256, 2
    cfg = M.MoEConfig(hidden=128, ffn=256, num_experts=E, topk=k, tokens=T)
    busiest = {}
    for nshadow in (0, 3):
        heaps = SymmetricHeap.emulated(W, 48 << 20)
        try:
            with cpu_kernel_model.installed():
                layers = [MoELayer(cfg, heaps[r], r, W, device="cpu", seed=2, name="l", shadow_experts=nshadow) for r in range(W)]
                for r in range(1, W):
                    layers[r].router.data.copy_(layers[0].router.data)
                g = torch.Generator().manual_seed(7)
                for r in range(W):
                    x = torch.randn(T, 128, generator=g).to(torch.bfloat16)
                    M.moe_forward_dispatch(layers[r].ws, x, layers[r].route(x)[1].contiguous())
                rows = [int(l.ws.counts_now().sum()) for l in layers]
                assert sum(rows) == W * T * k
                busiest[nshadow] = max(rows)
        finally:
            for h in heaps:
                h.close()
    mean = T * k
    assert busiest[0] > 2.2 * mean and busiest[3] < 1.5 * mean, busiest


def test_autograd_node_returns_gradients_for_experts_and_copies():
    """MoEFunction end to end (one rank): with expert 2 shadowed its gradient arrives in the copy's slot and the idle slot of
    the expert itself gets zeros; everything equals the plain-PyTorch path of the same layer."""
    import cpu_kernel_model
    from fuselink_b200.models.moe import MoELayer
    from fuselink_b200.ops import moe as M
    from fuselink_b200.parallel.symm import SymmetricHeap
    E, T, k, H = 4, 48, 2, 128
    cfg = M.MoEConfig(hidden=H, ffn=256, num_experts=E, topk=k, tokens=T)
    heaps = SymmetricHeap.emulated(1, 32 << 20)
    try:
        with cpu_kernel_model.installed():
            layer = MoELayer(cfg, heaps[0], 0, 1, device="cpu", seed=6, name="a", shadow_experts=[2])
            x = torch.randn(T, H).to(torch.bfloat16)
            xa, xb = x.clone().requires_grad_(True), x.clone().requires_grad_(True)
            w, idx = layer.route(xa)
            out = M.MoEFunction.apply(xa, w, idx, layer.w13, layer.w2, layer.ws, 0.0)
            out.float().pow(2).sum().backward()
            got13, got2, gotx = layer.w13.grad.clone(), layer.w2.grad.clone(), xa.grad.clone()
            layer.zero_grad(set_to_none=True)
            wb, idxb = layer.route(xb)
            layer._forward_reference(xb, wb, idxb).float().pow(2).sum().backward()
            want13, want2 = layer.w13.grad, layer.w2.grad                      # plain path: gradients in the experts' own slots
        close = lambda a, b: (a.float() - b.float()).abs().max().item() < 4e-2 * (b.float().abs().max().item() + 1e-6)
        assert got13.shape[0] == E + 1 and close(gotx, xb.grad)
        for e in (0, 1, 3):
            assert close(got13[e], want13[e]) and close(got2[e], want2[e])
        assert close(got13[E], want13[2]) and close(got2[E], want2[2])          # the copy carries expert 2's gradient
        assert got13[2].abs().max() == 0 and got2[2].abs().max() == 0           # expert 2's own slot saw no rows
    finally:
        heaps[0].close()


def test_changing_the_shadowed_expert_between_steps():
    """Step with expert 0 shadowed, then with expert 5 instead (same slot, other table, weights moved): the forward result
    equals the oracle both times and the rows of the shadowed expert are the ones that stay local."""
    import dataclasses
    import cpu_kernel_model
    from fuselink_b200.models.moe import MoELayer
    from fuselink_b200.ops import gemm, moe as M, ref
    from fuselink_b200.parallel.symm import SymmetricHeap
    E, W, T, k, H = 8, 2, 48, 2, 128
    epr = E // W
    cfg = M.MoEConfig(hidden=H, ffn=256, num_experts=E, topk=k, tokens=T)
    heaps = SymmetricHeap.emulated(W, 48 << 20)
    try:
        with cpu_kernel_model.installed():
            layers = [MoELayer(cfg, heaps[r], r, W, device="cpu", zipf_s=None, seed=8, name="c", shadow_experts=[0]) for r in range(W)]
            for r in range(1, W):
                layers[r].router.data.copy_(layers[0].router.data)
            wg, wu = gemm.deinterleave_gate_up(torch.cat([l.w13.data[:epr] for l in layers]).float())
            w2 = torch.cat([l.w2.data[:epr] for l in layers]).float()
            for shadowed in (0, 5):
                if shadowed != layers[0].cfg.shadow[0]:
                    # what set_shadows does over a process group, done by hand for the ranks emulated in this process
                    for l in layers:
                        l.sync_shadow_to_real()
                    owner = layers[shadowed // epr]
                    for l in layers:
                        l.w13.data[epr].copy_(owner.w13.data[shadowed % epr])
                        l.w2.data[epr].copy_(owner.w2.data[shadowed % epr])
                        l.cfg = dataclasses.replace(l.cfg, shadow=(shadowed,))
                        l.ws.set_shadow((shadowed,))
                xs = [torch.randn(T, H).to(torch.bfloat16) for _ in range(W)]
                routes = [layers[r].route(xs[r]) for r in range(W)]
                for r in range(W):
                    M.moe_forward_dispatch(layers[r].ws, xs[r], routes[r][1].contiguous())
                for r in range(W):
                    local_rows = int((routes[r][1] == shadowed).sum())
                    assert int(layers[r].ws.counts_now()[epr]) == local_rows              # the copy slot holds this rank's own rows only
                    assert int(layers[r].ws.counts_now()[shadowed % epr]) == 0 or shadowed // epr != r
                for r in range(W):
                    M.moe_forward_experts(layers[r].ws, layers[r].w13.data, layers[r].w2.data)
                for r in range(W):
                    out = M.moe_forward_combine(layers[r].ws, routes[r][0].contiguous())
                    want = ref.moe_forward(xs[r].float(), routes[r][1], routes[r][0].float(), wg, wu, w2)
                    assert (out.float() - want).abs().max() < 3e-2 * (want.abs().max() + 1e-3)
                for h in heaps:
                    h.check_status("step")
    finally:
        for h in heaps:
            h.close()


def test_an_empty_copy_slot_costs_nothing_and_changes_nothing():
    """Two copy slots, one in use: same results as with exactly one slot, and the empty slot's gradient rows are zero."""
    _run_on_model(2, shadow=(4, -1))
    _run_on_model(2, sgd=0.05, steps=2, shadow=(4, -1))
    _run_on_model(2, shadow=(-1, -1))


@pytest.mark.parametrize("world,placement,shape,push", [(2, "", "", "1"), (2, "", "", "0"), (4, "", "", "1"), (2, "balanced", "", "1"),
                                                        (4, "balanced", "", "1"), (3, "balanced", "12 3 20", "1")])
def test_expert_parallel_step_between_processes(world, placement, shape, push, tmp_path):
    """Real processes over a shared-memory heap: forward, backward, the sum of the shadow experts' gradients over the ranks
    (pushed by the weight-gradient GEMMs to the rank that sums and updates each block of rows; an all-reduce with
    FUSELINK_PUSH_REDUCE=0, without the fused update, or when the rows do not divide over the ranks, as with 3 ranks here),
    the fused update, and a change of the shadowed experts by broadcast -- all against an fp32 autograd oracle."""
    import os
    import socket
    import subprocess
    import sys
    here = os.path.dirname(os.path.abspath(__file__))
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    env = dict(os.environ, FL_MODEL_LOCK=str(tmp_path / "reserve.lock"), FL_MOE_PLACEMENT=placement, FUSELINK_PUSH_REDUCE=push)
    if shape:                                                     # experts, top-k, tokens per rank (default 8, 2, 32)
        env.update(zip(("FL_MOE_E", "FL_MOE_K", "FL_MOE_T"), shape.split()))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(here, "mp_moe_cpu_worker.py")]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert out.stdout.count("MOE-MP-OK") == world, out.stdout[-2000:] + out.stderr[-4000:]


def test_moe_transformer_trains_between_processes(tmp_path):
    """Two processes, the MoE transformer with one shadowed expert per layer chosen again every step: replicated
    parameters and copies stay identical on both ranks and the loss falls."""
    import os
    import socket
    import subprocess
    import sys
    here = os.path.dirname(os.path.abspath(__file__))
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    env = dict(os.environ, FL_MODEL_LOCK=str(tmp_path / "reserve.lock"))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(here, "mp_moe_train_cpu_worker.py")]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert out.stdout.count("MOE-TRAIN-OK") == 2, out.stdout[-2000:] + out.stderr[-4000:]


@pytest.mark.parametrize("world", [3])
def test_dlrm_fused_step_between_processes(world):
    """Real processes, shared-memory heap, modelled embedding-bag entry points: losses, tables and dense weights follow the
    plain-PyTorch path of the same model step by step."""
    import os
    import socket
    import subprocess
    import sys
    here = os.path.dirname(os.path.abspath(__file__))
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(here, "mp_dlrm_cpu_worker.py")]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert out.stdout.count("DLRM-MP-OK") == world, out.stdout[-2000:] + out.stderr[-4000:]


def test_striped_transfer_over_relays_between_processes(tmp_path):
    """Four processes: the selector splits a 6 MiB transfer 0 -> 1 into a direct stripe and two relayed ones, the relays
    forward chunk by chunk as the source's flags appear, the destination gets every byte."""
    import os
    import socket
    import subprocess
    import sys
    here = os.path.dirname(os.path.abspath(__file__))
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    env = dict(os.environ, NCCL_FUSELINK_DEGREE="3", FUSELINK_MIN_STRIPE_BYTES="1048576", FL_MODEL_LOCK=str(tmp_path / "atomic.lock"))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=4", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(here, "mp_relay_cpu_worker.py")]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert out.stdout.count("RELAY-MP-OK") == 4, out.stdout[-2000:] + out.stderr[-4000:]


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
def test_online_serving_between_processes(dtype):
    """Trace -> scheduler -> prefill on one process, decode on another: paged KV, header, flags and pool credits over the
    shared heap (two pools used in turn, the end-of-trace header last); every generated token checked against the dense
    model.  fp32 also covers pools of 4-byte elements, which the KV entry point moves as heads twice as wide."""
    import os
    import socket
    import subprocess
    import sys
    here = os.path.dirname(os.path.abspath(__file__))
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(here, "mp_online_cpu_worker.py")]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=dict(os.environ, FL_ONLINE_DTYPE=dtype))
    assert out.stdout.count("ONLINE-MP-OK") == 2, out.stdout[-2000:] + out.stderr[-4000:]


def _run_script_on_model(script, args, nproc=1, env=None, timeout=600):
    import os
    import socket
    import subprocess
    import sys
    here = os.path.dirname(os.path.abspath(__file__))
    root = os.path.dirname(here)
    cmd = [os.path.join(here, "run_with_kernel_model.py"), os.path.join(root, script), *args]
    if nproc > 1:
        s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
        cmd = ["-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1", "--master-port", str(port)] + cmd
    out = subprocess.run([sys.executable, *cmd], capture_output=True, text=True, timeout=timeout, env=dict(os.environ, **(env or {})))
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-4000:]
    import json
    return [json.loads(l) for l in out.stdout.splitlines() if l.startswith("{")]


@pytest.mark.parametrize("nproc", [1, 4])
def test_online_serving_experiment_script_end_to_end(nproc):
    """experiments/run_online_serving.py itself: one process with both stages on an emulated heap, and four processes --
    two tensor-parallel prefill ranks, two decode ranks, the batches shared inside the prefill group."""
    rows = _run_script_on_model("experiments/run_online_serving.py", ["--device", "cpu", "--model", "tiny", "--requests", "12", "--rate", "300",
                                                                      "--input-len", "96", "--decode-steps", "2", "--policy", "sjf"], nproc=nproc)
    served = [r for r in rows if "served" in r]
    assert served and served[0]["served"] == 12
    assert sum(r["batch"] for r in rows if "batch" in r and "prompt_tokens" in r) == 12
    if nproc > 1:
        assert [r for r in rows if "decoded_requests" in r][0]["decoded_requests"] == 12


def test_moe_training_script_on_the_fused_path_between_processes(tmp_path):
    """experiments/run_moe_training.py itself, two processes, fused path on a host-memory heap: a shadowed expert per layer
    chosen again every step, the experts' update fused into the modelled wgrad, checkpoint and resume."""
    ck = str(tmp_path / "ck")
    env = {"FL_MODEL_LOCK": str(tmp_path / "atomic.lock")}
    base = ["--model", "tiny_moe", "--device", "cpu", "--host-heap", "--batch", "2", "--seq", "16", "--lr", "0.2", "--log-every", "1",
            "--shadow", "1", "--reshadow-every", "1"]
    rows = _run_script_on_model("experiments/run_moe_training.py", base + ["--steps", "3", "--checkpoint", ck], nproc=2, env=env)
    assert [r["step"] for r in rows] == [1, 2, 3] and all(r["n_gpus"] == 2 and 0 < r["loss"] < 20 for r in rows)
    import os
    assert os.path.exists(ck + ".rank0") and os.path.exists(ck + ".rank1")
    more = _run_script_on_model("experiments/run_moe_training.py", base + ["--steps", "1", "--resume", ck], nproc=2, env=env)
    fresh = _run_script_on_model("experiments/run_moe_training.py", base + ["--steps", "1"], nproc=2, env=env)
    assert fresh[0]["loss"] == rows[0]["loss"] and more[0]["loss"] != fresh[0]["loss"]      # the resumed run starts from trained weights


def test_dlrm_training_script_on_the_fused_path_between_processes():
    """experiments/run_dlrm_training.py, three processes (uneven table split), fused path on a host-memory heap: the losses
    are the ones of the plain path from the same seed."""
    args = ["--device", "cpu", "--tables", "5", "--rows", "300", "--global-batch", "96", "--pooling", "4", "--lr", "0.3", "--steps", "4", "--log-every", "1"]
    fused = _run_script_on_model("experiments/run_dlrm_training.py", args + ["--host-heap"], nproc=3)
    plain = _run_script_on_model("experiments/run_dlrm_training.py", args, nproc=3)
    assert [r["step"] for r in fused] == [1, 2, 3, 4]
    assert [r["loss"] for r in fused] == pytest.approx([r["loss"] for r in plain], abs=2e-5)


@pytest.mark.parametrize("pipeline", [True, False])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_offline_prefill_to_decode_on_the_model(pipeline, dtype):
    """The offline experiment's two stages as virtual ranks of one process: prefill with the per-layer (or one-shot) KV
    hand-off, then paged greedy decoding on the other side, against the dense model token by token."""
    import cpu_kernel_model
    from fuselink_b200.models.llama import MODEL_ZOO, LlamaShard
    from fuselink_b200.parallel.symm import SymmetricHeap
    from fuselink_b200.serving.disagg import DecodeStage, KVLink, PrefillStage, ServeParams, make_prompts
    p = ServeParams(model=MODEL_ZOO["tiny"], batch_size=3, input_len=64, num_decoding_step=4, dtype=dtype)
    heaps = SymmetricHeap.emulated(2, 32 << 20)
    try:
        with cpu_kernel_model.installed():
            net = LlamaShard(p.model, device="cpu", seed=1, dtype=dtype)
            links = [KVLink(h, p, net.kvh_local) for h in heaps]
            pre = PrefillStage(p, net, links[0], dst_rank=1, pipeline_layers=pipeline)
            dec = DecodeStage(p, net, links[1])
            prompts = make_prompts(p, "cpu", seed=3)
            rp = pre.run(prompts)
            rd = dec.run()
            for h in heaps:
                h.check_status()
        gen = rd.extra["generated"]
        assert gen.shape == (p.batch_size, 1 + p.num_decoding_step) and rd.extra["graph"] is False
        seq, agree = prompts.clone(), 0
        for t in range(1 + p.num_decoding_step):
            agree += int((net.forward_dense(seq).argmax(-1) == gen[:, t]).sum())
            seq = torch.cat([seq, gen[:, t:t + 1]], 1)
        total = p.batch_size * (1 + p.num_decoding_step)
        assert agree == total if dtype == torch.float32 else agree >= 0.8 * total
        assert rp.kv_bytes == 2 * p.batch_size * p.context_blocks_per_req * p.model.layers * links[0].page_elems * p.elem_bytes
        assert rd.tokens == p.batch_size * p.num_decoding_step
    finally:
        for h in heaps:
            h.close()


@pytest.mark.parametrize("nproc", [1, 4])
def test_serving_command_line_end_to_end(nproc):
    """`python -m fuselink_b200.serving` with the reference's flags (experiments/serving/main.cc:45-107): both stages on an
    emulated heap in one process, and 2 + 2 tensor-parallel ranks as four processes; fp32 pools."""
    rows = _run_script_on_model("fuselink_b200/serving/__main__.py",
                                ["--model_name", "tiny_opt", "--model_path", "dummy", "--precision", "fp32", "--input_len", "64", "--batch_size", "2",
                                 "--block_size", "16", "--num_decoding_step", "3", "--device", "cpu"], nproc=nproc)
    r = rows[-1]
    assert r["ttft_ms"] > 0 and r["decode_tok_s"] > 0 and r["prefill_ms"] > 0
    if nproc > 1:
        assert r["tp"] == 2 and r["n_gpus"] == 4 and 0 < r["comm_over_elapsed"] <= 1.0


def test_serving_command_line_replays_a_trace(tmp_path):
    from fuselink_b200.serving.tracegen import generate
    trace = tmp_path / "trace.txt"
    trace.write_text("\n".join(generate(requests=9, rate=500.0, prompt_min=16, prompt_max=60, seed=1)) + "\n")
    rows = _run_script_on_model("fuselink_b200/serving/__main__.py",
                                ["--model_name", "tiny", "--input_len", "64", "--num_decoding_step", "2", "--tracepath", str(trace), "--device", "cpu"])
    assert [r for r in rows if "served" in r][0]["served"] == 9


@pytest.mark.parametrize("nproc,extra", [(1, []), (2, ["--shadow", "1"]), (2, ["--placement", "contiguous", "--dtype", "fp8"])])
def test_headline_bench_script_plumbing(nproc, extra, tmp_path):
    """bench.py itself in its host mode under the model (tiny shape; not a measurement): warm-up, timed region, the
    end-to-end region, roofline block, one JSON line with every key the contract names, clean teardown -- on one process
    and on two, with a shadowed expert and with the fp8 arm."""
    rows = _run_script_on_model("bench.py", ["--device", "cpu", "--gpus", str(nproc), "--tokens", "64", "--hidden", "128", "--ffn", "256",
                                             "--steps", "2", "--warmup", "1", *extra], nproc=nproc, env={"FL_MODEL_LOCK": str(tmp_path / "atomic.lock")})
    assert len(rows) == 1
    r = rows[0]
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling", "vs_baseline", "dtype", "data",
                "config", "clocks", "e2e", "gpu_launches"):
        assert key in r, key
    assert r["n_gpus"] == nproc and r["steps"] == 2 and r["warmup"] == 1 and r["value"] > 0 and r["gpu_launches"] > 0
    assert r["config"]["global_batch"] == 64 * nproc and r["config"]["parallelism"].startswith(f"ep{nproc}")
    assert "error" not in r["e2e"] and r["e2e"]["value"] > 0 and r["e2e"]["h2d_bytes_per_step"] == 64 * 128 * 2
    assert "error" not in (r["roofline"] or {}) and r["roofline"]["hot_rank_rows"] >= r["roofline"]["mean_rows"] * (0.5 if extra[:1] == ["--shadow"] else 1.0)
    if extra[:1] == ["--shadow"]:
        assert "shadow experts [0]" in r["config"]["parallelism"]
    if nproc == 2:                                  # by default the experts' homes follow the load the router's bias predicts
        assert ("expert homes" in r["config"]["parallelism"]) == (extra[:1] != ["--placement"])
    if "--dtype" in extra:
        assert r["dtype"].startswith("fp8")


@pytest.mark.parametrize("nproc", [2])
def test_dlrm_bench_script_plumbing(nproc):
    rows = _run_script_on_model("bench/dlrm_bench.py", ["--device", "cpu", "--tables", "5", "--rows", "300", "--global-batch", "64", "--steps", "2",
                                                        "--warmup", "1"], nproc=nproc)
    r = rows[-1]
    assert r["n_gpus"] == nproc and r["value"] > 0 and 0.3 < r["loss"] < 1.2 and r["gpu_launches_per_step"] > 0


def test_variable_all_to_all_and_put_many_on_the_model():
    """ops/comm.py on four emulated ranks: a variable all-to-all with ragged blocks (one launch of up to 8 segments per
    rank, arrival counters derived from byte counts on both sides), twice, so the running totals are exercised too."""
    import cpu_kernel_model
    from fuselink_b200.ops.comm import Channel, all_to_all_v, chunking
    from fuselink_b200.parallel.symm import SymmetricHeap
    W = 4
    heaps = SymmetricHeap.emulated(W, 32 << 20)
    try:
        with cpu_kernel_model.installed():
            chans = [Channel(h, "v", engine="ldst") for h in heaps]
            cap = 3 << 20
            recvs = [h.alloc_tensor([W * cap], torch.uint8) for h in heaps]
            g = torch.Generator().manual_seed(0)
            for it in range(2):
                sizes = torch.randint(0, cap, (W, W), generator=g).tolist()          # sizes[r][p]: bytes r sends to p
                sizes[1][2] = 0                                                       # an empty block
                sends, offs = [], []
                for r in range(W):
                    o, acc = [], 0
                    for p in range(W):
                        o.append(acc)
                        acc += (sizes[r][p] + 15) // 16 * 16
                    offs.append(o)
                    sends.append(torch.randint(0, 255, (max(acc, 16),), dtype=torch.uint8, generator=g))
                for r in range(W):                                                    # every rank's launch, then every rank's wait
                    all_to_all_v(chans[r], sends[r], offs[r], sizes[r], recvs[r], [r * cap] * W, [sizes[p][r] for p in range(W)], wait=False)
                for r in range(W):
                    chans[r].wait()
                    heaps[r].check_status(f"a2a-v {it}")
                for r in range(W):
                    for p in range(W):
                        n = sizes[p][r]
                        assert torch.equal(recvs[r].local[p * cap: p * cap + n], sends[p][offs[p][r]: offs[p][r] + n]), (it, r, p)
            assert chunking(0)[1] == 0 and chunking(100)[1] == 1 and chunking(1 << 30)[0] == 512 * 1024
    finally:
        for h in heaps:
            h.close()


@pytest.mark.parametrize("world,placement,shadow,sgd", [(2, "balanced", (), 0.0), (4, "balanced", (), 0.0), (2, "balanced", (0,), 0.05),
                                                        (4, (7, 6, 5, 4, 3, 2, 1, 0), (), 0.05), (1, "balanced", (), 0.0)])
def test_expert_placement_on_the_model(world, placement, shadow, sgd):
    """Experts owned out of order (evened out by the router's bias, or any permutation): same outputs, gradients and updates
    as the oracle, which knows experts by id."""
    _run_on_model(world, placement=placement, shadow=shadow, sgd=sgd, steps=2 if sgd else 1)


@pytest.mark.parametrize("seed", range(8))
def test_random_moe_configurations_on_the_model(seed):
    """Ranks, experts, top-k, tokens, shadowed experts (with empty copy slots), placements (balanced or any permutation),
    fused update and the fp8 arm drawn at random from fixed seeds: every combination equals the oracle."""
    import random
    rng = random.Random(700 + seed)
    W = rng.choice([1, 2, 4])
    E = rng.choice([e for e in (4, 8, 16) if e % W == 0])
    nsh = rng.choice([0, 0, 1, 2])
    shadow = tuple(rng.sample(range(E), nsh)) + ((-1,) if nsh and rng.random() < 0.3 else ())
    placement = rng.choice([None, None, "balanced", tuple(rng.sample(range(E), E))])
    sgd = rng.choice([0.0, 0.05])
    import cpu_kernel_model
    from test_moe_gpu import _run
    with cpu_kernel_model.installed():
        _run(W, T=rng.choice([16, 48, 130]), H=128, Fd=256, E=E, k=rng.choice([1, 2, 3]), sgd=sgd, steps=2 if sgd else 1,
             fp8=rng.random() < 0.25, shadow=shadow, placement=placement, device="cpu")


def _default_step_trace(world, sgd, placement=None):
    """Every device call of two default MoE steps (no shadows, bf16), ranks emulated in one process."""
    import cpu_kernel_model
    from fuselink_b200.models.moe import MoELayer
    from fuselink_b200.ops import moe as M
    from fuselink_b200.parallel.symm import SymmetricHeap
    heaps = SymmetricHeap.emulated(world, 64 << 20)
    try:
        with cpu_kernel_model.installed() as model, cpu_kernel_model.recording(model, heaps[0].base, ) as trace:
            cfg = M.MoEConfig(hidden=128, ffn=256, num_experts=8, topk=2, tokens=48)
            layers = [MoELayer(cfg, heaps[r], r, world, device="cpu", seed=3, fused_sgd_lr=sgd, name="m", placement=placement) for r in range(world)]
            for step in range(2):
                g = torch.Generator().manual_seed(step)
                xs = [torch.randn(48, 128, generator=g).to(torch.bfloat16) for _ in range(world)]
                with torch.no_grad():
                    routes = [layers[r].route(xs[r]) for r in range(world)]
                wss = [l.ws for l in layers]
                for r in range(world):
                    M.moe_forward_dispatch(wss[r], xs[r], routes[r][1].contiguous())
                for r in range(world):
                    M.moe_forward_experts(wss[r], layers[r].w13.data, layers[r].w2.data)
                for r in range(world):
                    M.moe_forward_combine(wss[r], routes[r][0].contiguous())
                for r in range(world):
                    M.moe_backward_dispatch(wss[r], xs[r], routes[r][1].contiguous(), routes[r][0].contiguous())
                for r in range(world):
                    M.moe_backward_experts(wss[r], layers[r].w13.data, layers[r].w2.data, sgd, True)
                for r in range(world):
                    M.moe_backward_finish(wss[r], True)
        return trace
    finally:
        for h in heaps:
            h.close()


@pytest.mark.parametrize("world", [1, 2, 4])
@pytest.mark.parametrize("sgd", [0.0, 0.05])
def test_default_moe_step_hands_the_kernels_exactly_the_recorded_work(world, sgd):
    """The device calls of the default fused MoE step -- which entry point, in which order, with which scalars, tensor
    shapes, and addresses relative to the heap -- are pinned to a recorded digest, so an edit of the Python side that
    changes what the kernels are given (new options must leave the default alone) shows up here, on a machine without a
    GPU.  After a deliberate change of the default step the digests are recorded again: run this test with
    FUSELINK_RECORD_GOLDEN=1."""
    import hashlib
    import json
    import os
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "moe_default_step_calls.json")
    golden = json.load(open(path))
    trace = _default_step_trace(world, sgd)
    if os.environ.get("FUSELINK_RECORD_GOLDEN", "0") == "1":
        golden[f"world{world}_sgd{sgd}"] = {"calls": len(trace), "sha256": hashlib.sha256(json.dumps(trace).encode()).hexdigest()}
        json.dump(golden, open(path, "w"), indent=1)
        return
    want = golden[f"world{world}_sgd{sgd}"]
    assert len(trace) == want["calls"]
    assert hashlib.sha256(json.dumps(trace).encode()).hexdigest() == want["sha256"], "the default MoE step no longer issues the recorded device calls"


@pytest.mark.parametrize("world", [2, 4])
def test_placement_changes_nothing_the_kernels_can_see_but_index_values(world):
    """With the experts' homes evened out, a step issues the same device calls as in the recorded default -- same entry
    points, order, scalars, shapes and addresses; what differs are the values inside the index tensor and which expert's
    weights sit in which slot."""
    assert _default_step_trace(world, 0.05, placement="balanced") == _default_step_trace(world, 0.05)
    assert _default_step_trace(world, 0.05, placement=(7, 6, 5, 4, 3, 2, 1, 0)) == _default_step_trace(world, 0.05)


def test_push_reduce_falls_back_when_the_heap_has_no_room_or_the_rows_do_not_divide():
    """enable_push_reduce answers False, and the layer keeps ordinary tensors for its experts (the all-reduce formulation),
    when the symmetric heap cannot take the weights and the staging, and when the gradient rows do not divide over the
    ranks; with room and divisible rows the experts move onto the heap."""
    import os
    import cpu_kernel_model
    from fuselink_b200.models.moe import MoELayer
    from fuselink_b200.ops import moe as M
    from fuselink_b200.parallel.symm import SymmetricHeap
    cfg = M.MoEConfig(hidden=128, ffn=256, num_experts=4, topk=2, tokens=16)

    def on_heap(layer, heap):
        return heap.addr(0) <= layer.w13.data_ptr() < heap.addr(0) + heap.size

    with cpu_kernel_model.installed():
        heaps = SymmetricHeap.emulated(2, 32 << 20)
        three = SymmetricHeap.emulated(3, 32 << 20)
        try:
            # how much one workspace takes: push-reduce off
            os.environ["FUSELINK_PUSH_REDUCE"] = "0"
            try:
                before = heaps[0]._state["bump"]
                probe = MoELayer(cfg, heaps[0], 0, 2, device="cpu", seed=1, fused_sgd_lr=0.05, name="probe", shadow_experts=1)
                need = heaps[0]._state["bump"] - before
            finally:
                os.environ.pop("FUSELINK_PUSH_REDUCE", None)
            assert probe.ws.push is None and not on_heap(probe, heaps[0])
            # with room: the experts move onto the heap
            b = MoELayer(cfg, heaps[0], 0, 2, device="cpu", seed=1, fused_sgd_lr=0.05, name="b", shadow_experts=1)
            assert b.ws.push is not None and on_heap(b, heaps[0])
            assert b.w13.data_ptr() == b.ws.push.w13.addr() and b.w2.data_ptr() == b.ws.push.w2.addr()
            assert torch.equal(b.w13.detach(), probe.w13.detach())                       # same weights, new home
            # leave room for one more workspace and little else
            left = heaps[0].size - heaps[0]._state["bump"]
            heaps[0].alloc(left - need - (96 << 10))
            a = MoELayer(cfg, heaps[0], 0, 2, device="cpu", seed=1, fused_sgd_lr=0.05, name="a", shadow_experts=1)
            assert a.ws.push is None and not on_heap(a, heaps[0])
            # rows that do not divide over the ranks: 512 and 128 rows over 3 ranks
            odd = M.MoEConfig(hidden=128, ffn=256, num_experts=6, topk=2, tokens=16)
            c = MoELayer(odd, three[0], 0, 3, device="cpu", seed=1, fused_sgd_lr=0.05, name="c", shadow_experts=1)
            assert c.ws.push is None
        finally:
            for h in heaps + three:
                h.close()
