"""Block-scaled fp8 grouped GEMM: quantisers against their PyTorch restatement, and the GEMM against an fp32 matmul of
the DEQUANTISED operands (so the check isolates the kernel from the quantisation error)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _mk(shape, scale=1.0, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(*shape, generator=g, device="cuda") * scale).to(torch.bfloat16)


def _close(got, ref, tol=1.5e-2):
    if ref.numel() == 0:
        return
    err = (got.float() - ref).abs().max().item()
    den = ref.abs().max().item() + 1e-6
    assert err / den < tol, f"max abs err {err} vs ref max {den}"


def test_quantizers_match_reference():
    from fuselink_b200.ops import fp8
    x = _mk([300, 512], 3.0, seed=1)
    x[7] = 0
    q, s = fp8.quantize_rows(x)
    rq, rs = fp8.ref_quantize_rows(x)
    torch.testing.assert_close(s, rs, rtol=1e-6, atol=0)
    assert (q.float() - rq.float()).abs().max() <= 32            # at most one e4m3 step at the top of the range
    back = fp8.dequantize_rows(q, s)
    assert (back - x.float()).abs().max() <= 0.07 * x.float().abs().max()
    w = _mk([2, 256, 384], 0.05, seed=2)
    wq, ws = fp8.quantize_blocks(w)
    assert ws.shape == (2, 2, 3)
    wb = fp8.dequantize_blocks(wq, ws)
    assert (wb - w.float()).abs().max() <= 0.07 * w.float().abs().max()
    amax = w.float().view(2, 2, 128, 3, 128).abs().amax((2, 4))
    torch.testing.assert_close(ws, amax / 448.0, rtol=1e-6, atol=0)


@pytest.mark.parametrize("b_mn", [False, True])
@pytest.mark.parametrize("K", [128, 512])
def test_fp8_rows_store(K, b_mn):
    from fuselink_b200.ops import fp8
    G, cap, N = 3, 256, 512
    counts_l = [200, 0, 129]
    counts = torch.tensor(counts_l, dtype=torch.int32, device="cuda")
    a = _mk([G * cap, K], 2.0, seed=3)
    w = _mk([G, N, K], 0.1, seed=4)
    aq, asc = fp8.quantize_rows(a)
    if b_mn:
        wq, wsc = fp8.quantize_blocks(w.transpose(1, 2).contiguous())       # stored [G, K, N]
        wd = fp8.dequantize_blocks(wq, wsc).transpose(1, 2)
    else:
        wq, wsc = fp8.quantize_blocks(w)
        wd = fp8.dequantize_blocks(wq, wsc)
    ad = fp8.dequantize_rows(aq, asc)
    st = torch.zeros(8, dtype=torch.int32, device="cuda")
    out = torch.full((G * cap, N), 7.0, dtype=torch.bfloat16, device="cuda")
    fp8.grouped_gemm_rows_fp8(aq, asc, wq, wsc, counts, cap, b_mn_major=b_mn, out=out, zero_tail=True, status=st)
    torch.cuda.synchronize()
    assert st[0].item() == 0, st.tolist()
    for g, c in enumerate(counts_l):
        _close(out[g * cap:g * cap + c], ad[g * cap:g * cap + c] @ wd[g].t())
        end = min((c + 127) // 128 * 128, cap)
        assert (out[g * cap + c:g * cap + end] == 0).all()
        assert (out[g * cap + end:(g + 1) * cap] == 7.0).all()


def test_fp8_swiglu_scatter_and_dswiglu():
    import torch.nn.functional as F
    from fuselink_b200.ops import fp8, gemm
    G, cap, H, Fd = 2, 256, 256, 512
    counts_l = [256, 77]
    counts = torch.tensor(counts_l, dtype=torch.int32, device="cuda")
    x = _mk([G * cap, H], seed=5)
    w13 = gemm.interleave_gate_up(_mk([G, Fd, H], 0.1, seed=6), _mk([G, Fd, H], 0.1, seed=7))
    xq, xs = fp8.quantize_rows(x)
    wq, ws = fp8.quantize_blocks(w13)
    xd, wd = fp8.dequantize_rows(xq, xs), fp8.dequantize_blocks(wq, ws)
    st = torch.zeros(8, dtype=torch.int32, device="cuda")
    gu = torch.empty(G * cap, 2 * Fd, dtype=torch.bfloat16, device="cuda")
    act = fp8.grouped_gemm_rows_fp8(xq, xs, wq, ws, counts, cap, epilogue=fp8.EPI_SWIGLU, gu=gu, zero_tail=True, status=st)
    torch.cuda.synchronize()
    assert st[0].item() == 0
    for g, c in enumerate(counts_l):
        h = xd[g * cap:g * cap + c] @ wd[g].t()
        gate, up = gemm.deinterleave_gate_up(h.t().contiguous().unsqueeze(0))
        gate, up = gate[0].t(), up[0].t()
        _close(act[g * cap:g * cap + c], F.silu(gate) * up)
        gg, uu = gemm.deinterleave_gate_up(gu[g * cap:g * cap + c].t().contiguous().unsqueeze(0))
        _close(gg[0].t(), gate)
        _close(uu[0].t(), up)
    # second GEMM with the scatter epilogue
    w2 = _mk([G, H, Fd], 0.1, seed=8)
    aq, asc = fp8.quantize_rows(act)
    w2q, w2s = fp8.quantize_blocks(w2)
    dst = torch.zeros(G * cap, H, dtype=torch.bfloat16, device="cuda")
    info = torch.randperm(G * cap, device="cuda").int()
    fp8.grouped_gemm_rows_fp8(aq, asc, w2q, w2s, counts, cap, epilogue=fp8.EPI_SCATTER, row_info=info, peers=[dst.data_ptr()],
                              ldc=H, status=st)
    torch.cuda.synchronize()
    assert st[0].item() == 0
    ad, w2d = fp8.dequantize_rows(aq, asc), fp8.dequantize_blocks(w2q, w2s)
    for g, c in enumerate(counts_l):
        ref = ad[g * cap:g * cap + c] @ w2d[g].t()
        _close(dst[info[g * cap:g * cap + c].long()], ref)
    # backward of the activation: dAct = dY @ W2 (B MN-major), DSWIGLU epilogue
    dy = _mk([G * cap, H], seed=9)
    dyq, dys = fp8.quantize_rows(dy)
    dgu = torch.zeros_like(gu)
    fp8.grouped_gemm_rows_fp8(dyq, dys, w2q, w2s, counts, cap, b_mn_major=True, epilogue=fp8.EPI_DSWIGLU, gu=gu, dgu=dgu,
                              zero_tail=True, status=st)
    torch.cuda.synchronize()
    assert st[0].item() == 0
    dyd = fp8.dequantize_rows(dyq, dys)
    for g, c in enumerate(counts_l):
        da = dyd[g * cap:g * cap + c] @ w2d[g]
        gate, up = gemm.deinterleave_gate_up(gu[g * cap:g * cap + c].float().t().contiguous().unsqueeze(0))
        gate, up = gate[0].t(), up[0].t()
        sg = torch.sigmoid(gate)
        dg, du = gemm.deinterleave_gate_up(dgu[g * cap:g * cap + c].t().contiguous().unsqueeze(0))
        _close(dg[0].t(), da * up * (sg * (1 + gate * (1 - sg))), 2e-2)
        _close(du[0].t(), da * gate * sg, 2e-2)


def test_fp8_throughput_smoke():
    from fuselink_b200.ops import fp8
    cap, N, K = 8192, 4096, 4096
    aq, asc = fp8.quantize_rows(_mk([cap, K], seed=10))
    wq, wsc = fp8.quantize_blocks(_mk([1, N, K], 0.02, seed=11))
    st = torch.zeros(8, dtype=torch.int32, device="cuda")
    out = fp8.grouped_gemm_rows_fp8(aq, asc, wq, wsc, None, cap, status=st)
    torch.cuda.synchronize()
    assert st[0].item() == 0
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(10):
        fp8.grouped_gemm_rows_fp8(aq, asc, wq, wsc, None, cap, out=out, status=st)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / 10
    print(f"\n[fp8 gemm smoke] 8192x4096x4096 e4m3 1x128: {ms:.3f} ms  {2.0 * cap * N * K / ms / 1e9:.0f} TFLOP/s")
