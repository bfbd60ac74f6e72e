"""KV pack+send kernel and the disaggregated prefill -> decode path, both stages as virtual ranks on one GPU."""
import queue

import pytest
import torch

pytestmark = pytest.mark.gpu


def _setup(batch=3, input_len=64, steps=8, model="tiny"):
    from fuselink_b200.models.llama import MODEL_ZOO, LlamaShard
    from fuselink_b200.parallel.symm import SymmetricHeap
    from fuselink_b200.serving.disagg import KVLink, ServeParams
    p = ServeParams(model=MODEL_ZOO[model], batch_size=batch, input_len=input_len, num_decoding_step=steps)
    heaps = SymmetricHeap.emulated(2, 64 << 20)
    net = LlamaShard(p.model, device="cuda", seed=1)
    links = [KVLink(h, p, net.kvh_local) for h in heaps]
    return p, heaps, net, links


@pytest.mark.parametrize("same_layout", [False, True])
def test_kv_pack_send_matches_page_gather(same_layout):
    from fuselink_b200 import C
    from fuselink_b200.ops import ref
    L, H, S, D, B, maxb = 3, 2, 16, 64, 4, 5
    src_blocks, dst_blocks = 32, 40
    g = torch.Generator(device="cuda").manual_seed(0)
    page = H * S * D
    src_k = torch.randn(src_blocks * L * page, generator=g, device="cuda").to(torch.bfloat16)
    src_v = torch.randn(src_blocks * L * page, generator=g, device="cuda").to(torch.bfloat16)
    dst_k = torch.zeros(dst_blocks * L * page, dtype=torch.bfloat16, device="cuda")
    dst_v = torch.zeros_like(dst_k)
    nb = torch.tensor([5, 1, 0, 3], dtype=torch.int32, device="cuda")
    src_bt = torch.randperm(src_blocks, generator=torch.Generator().manual_seed(1))[:B * maxb].view(B, maxb).int().cuda()
    dst_bt = torch.randperm(dst_blocks, generator=torch.Generator().manual_seed(2))[:B * maxb].view(B, maxb).int().cuda()
    flag = torch.zeros(4, dtype=torch.int32, device="cuda")
    status = torch.zeros(8, dtype=torch.int32, device="cuda")
    counter = torch.zeros(1, dtype=torch.int32, device="cuda")
    hdr = torch.arange(10, dtype=torch.int64, device="cuda")
    hdr_dst = torch.zeros(10, dtype=torch.int64, device="cuda")
    dl = 0 if same_layout else 1
    for l0, l1, seq in [(0, 2, 1), (2, 3, 2)]:          # two launches: layers [0,2) then [2,3)
        C.kv_pack_send(src_k, src_v, dst_k.data_ptr(), dst_v.data_ptr(), 0, dl, src_blocks, dst_blocks, L, H, S, D, l0, l1,
                       src_bt, dst_bt, nb, hdr, hdr_dst.data_ptr(), flag.data_ptr(), seq, counter, 7, status.data_ptr())
    torch.cuda.synchronize()
    assert status[0].item() == 0 and flag[0].item() == 2 and counter.item() == 0
    assert torch.equal(hdr, hdr_dst)
    for src, dst in ((src_k, dst_k), (src_v, dst_v)):
        want = ref.kv_gather_pages(src, 0, src_bt.cpu(), nb.cpu(), L, H, S, D)
        got = ref.kv_gather_pages(dst, dl, dst_bt.cpu(), nb.cpu(), L, H, S, D)
        for w, g_ in zip(want, got):
            assert torch.equal(w, g_)
    # pages that were not addressed stay untouched
    used = set(int(dst_bt[b, j]) for b in range(B) for j in range(int(nb[b])))
    view = dst_k.view(L, dst_blocks, -1) if dl == 1 else dst_k.view(dst_blocks, L, -1).transpose(0, 1)
    for blk in range(dst_blocks):
        if blk not in used:
            assert (view[:, blk] == 0).all()


def test_kv_bad_block_id_is_reported_and_skipped():
    from fuselink_b200 import C
    L, H, S, D = 1, 1, 16, 64
    src = torch.ones(4 * L * H * S * D, dtype=torch.bfloat16, device="cuda")
    dst = torch.zeros(4 * L * H * S * D, dtype=torch.bfloat16, device="cuda")
    bt = torch.tensor([[0, 9]], dtype=torch.int32, device="cuda")           # 9 is outside the 4-page pools
    nb = torch.tensor([2], dtype=torch.int32, device="cuda")
    status = torch.zeros(8, dtype=torch.int32, device="cuda")
    counter = torch.zeros(1, dtype=torch.int32, device="cuda")
    C.kv_pack_send(src, src, dst.data_ptr(), dst.data_ptr(), 0, 0, 4, 4, L, H, S, D, 0, 1, bt, bt, nb, None, 0, 0, 1, counter, 2,
                   status.data_ptr())
    torch.cuda.synchronize()
    assert status[0].item() == 6                                              # kBadIndex: recorded, access skipped
    assert (dst.view(4, -1)[0] == 1).all() and (dst.view(4, -1)[1:] == 0).all()


@pytest.mark.parametrize("pipeline", [True, False])
def test_offline_prefill_to_decode_matches_dense_model(pipeline):
    from fuselink_b200.serving.disagg import DecodeStage, PrefillStage, make_prompts
    p, heaps, net, links = _setup()
    try:
        pre = PrefillStage(p, net, links[0], dst_rank=1, pipeline_layers=pipeline)
        dec = DecodeStage(p, net, links[1])
        prompts = make_prompts(p, "cuda", seed=3)
        rp = pre.run(prompts)
        rd = dec.run()
        for h in heaps:
            h.check_status()
        gen = rd.extra["generated"]                                           # [B, 1 + steps]
        assert gen.shape == (p.batch_size, 1 + p.num_decoding_step)
        # oracle: greedy decoding with the un-paged model, recomputing the full sequence each step
        seq = prompts.clone()
        for t in range(1 + p.num_decoding_step):
            nxt = net.forward_dense(seq).argmax(-1)
            agree = (nxt == gen[:, t]).float().mean().item()
            assert agree == 1.0, f"token {t}: paged path disagrees with the dense model ({agree:.2f})"
            seq = torch.cat([seq, gen[:, t:t + 1]], 1)
        assert rp.kv_bytes == 2 * p.batch_size * p.context_blocks_per_req * p.model.layers * links[0].page_elems * 2
        assert rp.kv_ms > 0 and rd.tokens == p.batch_size * p.num_decoding_step
    finally:
        for h in heaps:
            h.close()


def test_online_trace_batches_with_pool_credits():
    from fuselink_b200.models.llama import MODEL_ZOO, LlamaShard
    from fuselink_b200.parallel.symm import SymmetricHeap
    from fuselink_b200.serving.disagg import KVLink, ServeParams
    from fuselink_b200.serving.online import OnlineDecode, OnlinePrefill, TraceReader, next_batch, parse_trace
    p = ServeParams(model=MODEL_ZOO["tiny"], batch_size=20, input_len=96, num_decoding_step=4)
    heaps = SymmetricHeap.emulated(2, 96 << 20)
    try:
        net = LlamaShard(p.model, device="cuda", seed=1)
        links = [[KVLink(h, p, net.kvh_local, name=f"kv{i}") for i in range(2)] for h in heaps]
        pre = OnlinePrefill(p, net, links[0], dst_rank=1)
        dec = OnlineDecode(p, net, links[1], src_rank=0)
        trace = [f"ts: {0.001 * i:.3f} prompt: {40 + 7 * (i % 9)} shared: {3 * (i % 4)} out: {5 + i % 3}" for i in range(30)]
        trace.append("ts: 0.030 prompt: 5000 shared: 0 out: 4")               # longer than input_len: must be dropped, not spin
        reqs = parse_trace(trace)
        assert len(reqs) == 31 and reqs[1].active_prompt_len == 47 - 3
        q = queue.Queue()
        TraceReader(reqs, q, time_scale=1.0).start()
        warnings, served, finished = [], 0, False
        while not finished:
            batch, finished = next_batch(q, 20, p.input_len, warnings.append)
            if not batch:
                continue
            st = pre.serve_batch(batch)
            out = dec.serve_batch(max_steps=3)
            assert out["batch"] == len(batch) == st.batch
            assert out["generated"].shape == (len(batch), 4)
            bs = p.model.block_size
            want_pages = sum((r.active_prompt_len + bs - 1) // bs for r in batch)
            assert st.kv_bytes == want_pages * p.model.layers * links[0][0].page_elems * 4   # padding is never sent
            served += len(batch)
        assert served == 30 and len(warnings) == 1
        assert pre.batches >= 2                                               # pools were reused through the credit word
        for h in heaps:
            h.check_status()
    finally:
        for h in heaps:
            h.close()
