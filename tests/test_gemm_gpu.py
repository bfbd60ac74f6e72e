"""tcgen05 grouped GEMM against a plain fp32 PyTorch restatement (small shapes, every operand layout and
every fused epilogue)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True, params=["single", "pair", "wide"])
def _variant(request):
    """Every test runs on the three kernels: one CTA per 128x256 tile, CTA pairs on 256x256 tiles (cta_group::2, two
    accumulators), and CTA pairs on 256x512 tiles (one accumulator handed back in halves)."""
    from fuselink_b200 import C
    before = C.gemm_get_variant()
    C.gemm_set_variant({"single": 0, "pair": 1, "wide": 2}[request.param])
    yield request.param
    C.gemm_set_variant(before)


def _mk(shape, scale=1.0, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(*shape, generator=g, device="cuda") * scale).to(torch.bfloat16)


def _status():
    return torch.zeros(8, dtype=torch.int32, device="cuda")


def _check_status(st):
    v = st.cpu().tolist()
    assert v[0] == 0, f"kernel reported status {v}"


def _close(got, ref, tol=2e-2):
    if ref.numel() == 0:
        return
    err = (got.float() - ref).abs().max().item()
    den = ref.abs().max().item() + 1e-6
    assert err / den < tol, f"max abs err {err} vs ref max {den}"


@pytest.mark.parametrize("K", [64, 192, 136, 1024])
@pytest.mark.parametrize("b_mn", [False, True])
def test_rows_store(K, b_mn):
    from fuselink_b200.ops import gemm
    G, cap, N = 3, 256, 512
    counts = torch.tensor([200, 0, 129], dtype=torch.int32, device="cuda")
    a = _mk([G * cap, K], seed=1)
    w = _mk([G, N, K], 0.1, seed=2)            # logical B_g[N, K]
    b = w.transpose(1, 2).contiguous() if b_mn else w
    st = _status()
    out = torch.full((G * cap, N), 7.0, dtype=torch.bfloat16, device="cuda")
    gemm.grouped_gemm_rows(a, b, counts, cap, b_mn_major=b_mn, out=out, zero_tail=True, status=st)
    torch.cuda.synchronize()
    _check_status(st)
    for g in range(G):
        c = int(counts[g])
        ref = a[g * cap:g * cap + c].float() @ w[g].float().t()
        _close(out[g * cap:g * cap + c], ref)
        tail_end = min((c + 127) // 128 * 128, cap)
        assert (out[g * cap + c:g * cap + tail_end] == 0).all(), "tail rows must be zeroed"
        assert (out[g * cap + tail_end:(g + 1) * cap] == 7.0).all(), "rows past the tail must be untouched"


def test_rows_many_tiles_multi_cta_order():
    from fuselink_b200.ops import gemm
    G, cap, N, K = 2, 1024, 1024, 512
    counts = torch.tensor([1024, 700], dtype=torch.int32, device="cuda")
    a = _mk([G * cap, K], seed=3)
    w = _mk([G, N, K], 0.05, seed=4)
    st = _status()
    out = gemm.grouped_gemm_rows(a, w, counts, cap, status=st, group_m=4)
    torch.cuda.synchronize()
    _check_status(st)
    for g in range(G):
        c = int(counts[g])
        _close(out[g * cap:g * cap + c], a[g * cap:g * cap + c].float() @ w[g].float().t())


def test_wgrad_and_fused_sgd():
    from fuselink_b200.ops import gemm
    G, cap, M, N = 3, 256, 256, 512
    counts_l = [200, 0, 129]
    counts = torch.tensor(counts_l, dtype=torch.int32, device="cuda")
    a = _mk([G * cap, M], seed=5)
    b = _mk([G * cap, N], seed=6)
    for g, c in enumerate(counts_l):           # rows past the count are zero up to the 128-row tile edge
        a[g * cap + c:(g + 1) * cap] = 0
        b[g * cap + c:g * cap + (c + 127) // 128 * 128] = 0
    st = _status()
    dw = gemm.grouped_gemm_wgrad(a, b, counts, cap, G, status=st)
    torch.cuda.synchronize()
    _check_status(st)
    refs = []
    for g, c in enumerate(counts_l):
        ref = a[g * cap:g * cap + c].float().t() @ b[g * cap:g * cap + c].float()
        refs.append(ref)
        if c == 0:
            assert (dw[g] == 0).all()
        else:
            _close(dw[g], ref)
    w = _mk([G, M, N], seed=7)
    w0 = w.clone()
    gemm.grouped_gemm_wgrad(a, b, counts, cap, G, out=w, sgd_lr=0.01, status=st)
    torch.cuda.synchronize()
    _check_status(st)
    for g in range(G):
        _close(w[g], w0[g].float() - 0.01 * refs[g], tol=1e-2)


def test_swiglu_and_backward_epilogues():
    from fuselink_b200.ops import gemm
    import torch.nn.functional as F
    G, cap, H, Fd = 2, 256, 256, 512
    counts_l = [256, 77]
    counts = torch.tensor(counts_l, dtype=torch.int32, device="cuda")
    x = _mk([G * cap, H], seed=8)
    wg = _mk([G, Fd, H], 0.1, seed=9)
    wu = _mk([G, Fd, H], 0.1, seed=10)
    w13 = gemm.interleave_gate_up(wg, wu)
    g2, u2 = gemm.deinterleave_gate_up(w13)
    assert torch.equal(g2, wg) and torch.equal(u2, wu)
    st = _status()
    gu = torch.empty(G * cap, 2 * Fd, dtype=torch.bfloat16, device="cuda")
    act = gemm.grouped_gemm_rows(x, w13, counts, cap, epilogue=gemm.EPI_SWIGLU, gu=gu, zero_tail=True, status=st)
    torch.cuda.synchronize()
    _check_status(st)
    dact = _mk([G * cap, Fd], seed=11)
    for g, c in enumerate(counts_l):
        xs = x[g * cap:g * cap + c].float()
        gate, up = xs @ wg[g].float().t(), xs @ wu[g].float().t()
        _close(act[g * cap:g * cap + c], F.silu(gate) * up)
        gg, uu = gemm.deinterleave_gate_up(gu[g * cap:g * cap + c].t().contiguous().unsqueeze(0))
        _close(gg[0].t(), gate)
        _close(uu[0].t(), up)
    # DSWIGLU: accumulator = dAct = dY @ W2 with W2 given as [G, K=H2, N=Fd] (MN-major B)
    H2 = 128
    dy = _mk([G * cap, H2], seed=12)
    w2 = _mk([G, H2, Fd], 0.1, seed=13)        # nn.Linear layout of the down projection: [out=H2, in=Fd]
    dgu = torch.zeros_like(gu)
    gemm.grouped_gemm_rows(dy, w2, counts, cap, b_mn_major=True, epilogue=gemm.EPI_DSWIGLU, gu=gu, dgu=dgu,
                           zero_tail=True, status=st)
    torch.cuda.synchronize()
    _check_status(st)
    for g, c in enumerate(counts_l):
        da = dy[g * cap:g * cap + c].float() @ w2[g].float()
        gsl = gu[g * cap:g * cap + c].float()
        gate, up = gemm.deinterleave_gate_up(gsl.t().contiguous().unsqueeze(0))
        gate, up = gate[0].t(), up[0].t()
        sg = torch.sigmoid(gate)
        ref_dg = da * up * (sg * (1 + gate * (1 - sg)))
        ref_du = da * gate * sg
        dg, du = gemm.deinterleave_gate_up(dgu[g * cap:g * cap + c].t().contiguous().unsqueeze(0))
        _close(dg[0].t(), ref_dg)
        _close(du[0].t(), ref_du)


def test_scatter_epilogue_to_peer_slots():
    from fuselink_b200.ops import gemm
    G, cap, N, K, world = 2, 128, 256, 128, 3
    counts_l = [128, 50]
    counts = torch.tensor(counts_l, dtype=torch.int32, device="cuda")
    a = _mk([G * cap, K], seed=14)
    w = _mk([G, N, K], 0.1, seed=15)
    nslots = 200
    bufs = [torch.zeros(nslots, N, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    gen = torch.Generator().manual_seed(0)
    perm = torch.randperm(world * nslots, generator=gen)[:G * cap]
    rank, slot = (perm // nslots).int(), (perm % nslots).int()
    info = ((rank << 28) | slot).int().cuda()
    st = _status()
    gemm.grouped_gemm_rows(a, w, counts, cap, epilogue=gemm.EPI_SCATTER, row_info=info,
                           peers=[b.data_ptr() for b in bufs], ldc=N, status=st)
    torch.cuda.synchronize()
    _check_status(st)
    touched = torch.zeros(world, nslots, dtype=torch.bool)
    for g, c in enumerate(counts_l):
        ref = a[g * cap:g * cap + c].float() @ w[g].float().t()
        for i in range(c):
            r, s = int(rank[g * cap + i]), int(slot[g * cap + i])
            touched[r, s] = True
            _close(bufs[r][s], ref[i])
    for r in range(world):
        assert (bufs[r][~touched[r].cuda()] == 0).all(), "rows that were not routed must stay untouched"


def test_throughput_smoke():
    """Not a benchmark: checks that a production-sized launch completes and reports its rate."""
    from fuselink_b200.ops import gemm
    G, cap, N, K = 1, 8192, 4096, 4096
    a = _mk([G * cap, K], seed=16)
    w = _mk([G, N, K], 0.02, seed=17)
    st = _status()
    out = gemm.grouped_gemm_rows(a, w, None, cap, status=st)
    torch.cuda.synchronize()
    _check_status(st)
    ref = a[:256].float() @ w[0].float().t()
    _close(out[:256], ref)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(3):
        gemm.grouped_gemm_rows(a, w, None, cap, out=out, status=st)
    e0.record()
    for _ in range(10):
        gemm.grouped_gemm_rows(a, w, None, cap, out=out, status=st)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / 10
    tf = 2.0 * cap * N * K / ms / 1e9
    print(f"\n[gemm smoke] 8192x4096x4096 bf16: {ms:.3f} ms  {tf:.0f} TFLOP/s")
    assert tf > 50, "tensor-core path is not being used"


@pytest.mark.parametrize("world,M,lr", [(2, 512, 0.5), (4, 1024, 0.5), (2, 384, 0.0), (8, 2048, 0.25), (3, 768, 0.5)])
def test_wgrad_push_and_update_sum_the_ranks_partials(world, M, lr):
    """The two halves of the sum of replicated experts' weight gradients, with the ranks emulated one after the other on
    this GPU (neither kernel waits for another): every rank's GEMM deals its result rows out to the staging of the rank
    that sums them, then every rank sums its blocks, updates them and writes them into every copy.  Against fp32:
    w - lr * sum over ranks of A_r^T B_r (or the sum itself), identical in every copy."""
    from fuselink_b200.ops import gemm
    G, cap, N = 2, 512, 256
    blk = gemm.push_block_log2(M, world)
    assert blk >= 0
    counts = [torch.tensor([300 - 17 * r, 37 * (r % 2)], dtype=torch.int32, device="cuda") for r in range(world)]
    a = [_mk([G * cap, M], seed=10 + r) for r in range(world)]
    b = [_mk([G * cap, N], seed=50 + r) for r in range(world)]
    for r in range(world):          # the contraction runs over whole 64-row blocks: rows past the count are zero, as the MoE step leaves them
        for g in range(G):
            c = int(counts[r][g])
            a[r][g * cap + c:g * cap + (c + 127) // 128 * 128] = 0
            b[r][g * cap + c:g * cap + (c + 127) // 128 * 128] = 0
    stage = [torch.full((G, world, M // world, N), 3.0, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    w0 = _mk([G, M, N], 0.5, seed=99)
    copies = [w0.clone() for _ in range(world)]
    outs = copies if lr else [torch.full_like(w0, 5.0) for _ in range(world)]
    st = _status()
    for r in range(world):
        gemm.grouped_gemm_wgrad_push(a[r], b[r], counts[r], cap, G, [s.data_ptr() for s in stage], r, blk, status=st)
    for r in range(world):
        gemm.shadow_update(stage[r], copies[r] if lr else None, [o.data_ptr() for o in outs], G, r, M, N, blk, M * N, lr)
    torch.cuda.synchronize()
    _check_status(st)
    for g in range(G):
        total = sum(a[r][g * cap:g * cap + int(counts[r][g])].float().t() @ b[r][g * cap:g * cap + int(counts[r][g])].float()
                    for r in range(world))
        ref = w0[g].float() - lr * total if lr else total
        err = (outs[0][g].float() - ref).abs().max().item()
        # every rank's partial is rounded to bf16 once, the result once
        assert err < 2e-2 * (total.abs().max().item() * (lr or 1.0)) + 4e-3 * ref.abs().max().item(), (g, err)
    for r in range(1, world):
        assert torch.equal(outs[r], outs[0]), "every copy holds the same bits"


def test_wgrad_push_rejects_rows_that_do_not_divide_over_the_ranks():
    from fuselink_b200.ops import gemm
    a, b = _mk([256, 384], seed=1), _mk([256, 256], seed=2)
    counts = torch.tensor([100], dtype=torch.int32, device="cuda")
    stage = torch.zeros(1, 2, 192, 256, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError):
        gemm.grouped_gemm_wgrad_push(a, b, counts, 256, 1, [stage.data_ptr()] * 2, 0, 8)      # 384 rows: not 2 x 256
    with pytest.raises(RuntimeError):
        gemm.grouped_gemm_wgrad_push(a, b, counts, 256, 1, [stage.data_ptr()] * 2, 2, 6)      # rank 2 of 2
