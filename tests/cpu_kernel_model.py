"""A functional model, in plain PyTorch on host memory, of the device entry points the fused paths call: the MoE step
(`moe_dispatch`, `moe_zero_tail`, `grouped_gemm` with its five epilogues, `moe_combine`, `moe_combine_dw`, the fp8 quantisers
and the block-scaled fp8 grouped GEMM), the DLRM step (`embbag` forward and backward), the KV hand-off of serving
(`kv_pack_send`) and the transfers (`put_chunks`, `all_to_all`, `wait_flags`, `barrier`).

It takes the same arguments as the bindings of the real extension, raw addresses of peers' buffers included, and does to
the memory behind them what the kernels are specified to do.  With it the Python side of the fused paths -- buffer sizes,
slices, parities, the order of the phases, which barrier protects what, what is handed to which call -- runs on a machine
without a GPU, over a symmetric heap that lives in host memory: ranks emulated in one process (`SymmetricHeap.emulated`
on the memfd backend), or real processes that share the regions (`SymmetricHeap.create(device=-1)`), in which case waits
and barriers are real and bounded like the kernels'.  It says nothing about the kernels themselves; those are tested on
the GPU against the same fp32 oracles.

Use: ``with cpu_kernel_model.installed(): ...`` replaces ``require_native`` in the modules of those paths.
"""
import contextlib

import torch

EPI_STORE, EPI_SWIGLU, EPI_SCATTER, EPI_DSWIGLU, EPI_WGRAD = 0, 1, 2, 3, 4


class Model:
    """Everything that is not modelled (the cuMem layer, tensor_from_ptr, ...) is the real extension's."""

    def __init__(self, real):
        self._real = real

    def __getattr__(self, name):
        return getattr(self._real, name)

    def _view(self, addr, shape, dtype):
        return self._real.tensor_from_ptr(int(addr), list(shape), dtype, -1)

    def _status(self, status_addr, code, where):
        st = self._view(status_addr, [8], torch.int32)
        if st[0] == 0:
            st[0], st[1] = code, where

    # ---------------------------------------------------------------------------------------- flags, copies, barrier
    # Ranks emulated in ONE process run their phases one after the other, so a wait finds its flags already set.  Ranks
    # that are separate processes over a shared-memory heap (SymmetricHeap.create on the memfd backend) really wait here,
    # with the kernels' rule: a wait that runs out records a status and returns.
    wait_limit_s = 2.0

    def _flag(self, addr):
        return self._view(addr, [1], torch.int32)

    def _wait_ge(self, addr, want, status_addr, where):
        import time
        f = self._flag(addr)
        t0 = time.monotonic()
        while ((int(f[0]) - int(want)) & 0xFFFFFFFF) >= 0x80000000:          # wrap-around "less than"
            if time.monotonic() - t0 > self.wait_limit_s:
                self._status(status_addr, 1, where)
                return False
            time.sleep(0.0002)
        return True

    def barrier(self, pads, slot0, rank, world, seq, do_signal, do_wait, status_addr):
        if do_signal:
            for r in range(world):
                self._flag(pads[r] + 4 * (slot0 + rank))[0] = int(seq) - (1 << 32 if int(seq) >= (1 << 31) else 0)
        if do_wait and not self.single_process:
            for r in range(world):
                self._wait_ge(pads[rank] + 4 * (slot0 + r), seq, status_addr, 800 + r)

    single_process = True
    lock_path = None                 # ranks in separate processes: a file all of them lock around a reservation

    @contextlib.contextmanager
    def _reserve_lock(self):
        if self.single_process or not self.lock_path:
            yield
            return
        import fcntl
        with open(self.lock_path, "a") as f:
            fcntl.flock(f, fcntl.LOCK_EX)
            try:
                yield
            finally:
                fcntl.flock(f, fcntl.LOCK_UN)

    def put_chunks(self, segs, chunk_bytes, seq, use_bulk, num_ctas, threads, status_addr, counters=(), counter_scratch=0):
        for i, (src, dst, nbytes, flags, mode, wait_flags) in enumerate(segs):
            nchunks = (nbytes + chunk_bytes - 1) // chunk_bytes
            for c in range(nchunks):
                off = c * chunk_bytes
                n = min(chunk_bytes, nbytes - off)
                if wait_flags and not self._wait_ge(wait_flags + 4 * c, seq, status_addr, 600 + i):
                    return                                                    # a relay forwards a chunk once its flag shows this transfer
                self._view(dst + off, [n], torch.uint8).copy_(self._view(src + off, [n], torch.uint8))
                if mode == 2:                                                 # arrival counter: one per chunk, several senders
                    with self._reserve_lock():                                # (the kernel's red.release.sys.add)
                        f = self._flag(flags)
                        f[0] = ((int(f[0]) + 1 + (1 << 31)) % (1 << 32)) - (1 << 31)
                elif mode == 1:                                               # one word per chunk = seq
                    self._flag(flags + 4 * c)[0] = int(seq)
                if i < len(counters) and counters[i]:
                    self._view(counters[i], [1], torch.int64)[0] += n

    def wait_flags(self, flags, status_addr, limit_ms=0):
        for i, (addr, want) in enumerate(flags):
            self._wait_ge(addr, want, status_addr, 700 + i)

    def all_to_all(self, send_addr, recv_peers, per, rank, pads, slot0, chunk_bytes, want, use_bulk, num_ctas, threads, status_addr):
        world = len(recv_peers)
        segs = [(send_addr + p * per, recv_peers[p] + rank * per, per, pads[p] + 4 * (slot0 + rank), 2, 0)
                for p in ((rank + k) % world for k in range(world))]
        self.put_chunks(segs, chunk_bytes, 0, use_bulk, num_ctas, threads, status_addr)
        for r, w in enumerate(want):
            self._wait_ge(pads[rank] + 4 * (slot0 + r), w, status_addr, 600 + r)

    # ---------------------------------------------------------------------------------------- KV pack + send
    def kv_pack_send(self, src_k, src_v, dst_k, dst_v, src_layout, dst_layout, src_blocks, dst_blocks, L, H, S, D, l0, l1,
                     src_bt, dst_bt, nblocks, hdr, hdr_dst, done_flag, seq, cta_counter, num_ctas, status_addr):
        """Pages named by the block tables go from the local pools into the peer's, layers [l0, l1), with the change of
        layout (0 = [block][layer][head][slot][dim], 1 = [layer][block][slot][head][dim]; elements of 2 bytes); then the
        header, then the flag."""
        def pool(t_or_addr, nblk, layout):
            n = nblk * L * H * S * D                                  # the pool may be larger than the pages this call names
            flat = t_or_addr.view(torch.int16).view(-1)[:n] if torch.is_tensor(t_or_addr) else self._view(t_or_addr, [n], torch.int16)
            return flat.view(nblk, L, H, S, D) if layout == 0 else flat.view(L, nblk, S, H, D)

        def page(p, layout, blk, layer):                         # always as [head][slot][dim]
            return p[blk, layer] if layout == 0 else p[layer, blk].transpose(0, 1)

        for src, dst in ((src_k, dst_k), (src_v, dst_v)):
            sp, dp = pool(src, src_blocks, src_layout), pool(dst, dst_blocks, dst_layout)
            for b in range(src_bt.shape[0]):
                for j in range(int(nblocks[b])):
                    sb, db = int(src_bt[b, j]), int(dst_bt[b, j])
                    if not (0 <= sb < src_blocks and 0 <= db < dst_blocks):
                        self._status(status_addr, 6, 1000)
                        continue
                    for layer in range(l0, l1):
                        page(dp, dst_layout, db, layer).copy_(page(sp, src_layout, sb, layer))
        if hdr is not None and hdr_dst:
            raw = hdr.contiguous().view(torch.uint8).view(-1)
            self._view(hdr_dst, [raw.numel()], torch.uint8).copy_(raw)
        if done_flag:
            self._flag(done_flag)[0] = int(seq)

    # ---------------------------------------------------------------------------------------- embedding bag + all-to-all
    def embbag(self, backward, weights, indices, t_first, t_total, b_local, peers, lr, num_ctas, status_addr):
        """forward: the pooled vector of (local table t, global sample b) is stored into the sample owner's
        [b_local, t_total, dim] buffer; backward: the gradient is read from there and every pooled row gets -lr * grad."""
        assert weights.dtype == torch.float32 and indices.dtype == torch.int64 and indices.shape[0] == weights.shape[0]
        T, rows, dim = weights.shape
        _, B, pooling = indices.shape
        if ((indices < 0) | (indices >= rows)).any():
            self._status(status_addr, 6, 900)
        idx = indices.clamp(0, rows - 1)
        bufs = [self._view(p, [b_local, t_total, dim], torch.float32) for p in peers]
        for t in range(T):
            for owner in range(B // b_local):
                sl = slice(owner * b_local, (owner + 1) * b_local)
                if not backward:
                    bufs[owner][:, t_first + t] = weights[t][idx[t, sl]].sum(1)
                else:
                    g = bufs[owner][:, t_first + t]                                    # [b_local, dim]
                    weights[t].index_add_(0, idx[t, sl].reshape(-1), (-lr * g).repeat_interleave(pooling, 0))

    # ---------------------------------------------------------------------------------------- dispatch
    def moe_dispatch(self, x, topk_idx, row_scale, num_experts, epr, cap, rank, world, local_count, base, pos, slot,
                     count_peers, parity, x_peers, info_peers, reuse, status_addr):
        assert x.dtype == torch.bfloat16 and x.is_contiguous() and topk_idx.dtype == torch.int32 and topk_idx.is_contiguous()
        assert epr * world == num_experts and local_count.numel() >= num_experts and base.numel() >= num_experts
        T, k = topk_idx.shape
        H = x.shape[1]
        idx = topk_idx.view(-1)
        posf, slotf = pos.view(-1), slot.view(-1)
        if not reuse:
            for i in range(T * k):
                e = int(idx[i])
                if e < 0 or e >= num_experts:
                    self._status(status_addr, 6, 1100)
                    posf[i] = -1
                    continue
                posf[i] = local_count[e]
                local_count[e] += 1
            with self._reserve_lock():                              # what atomicAdd_system gives the kernel
                for e in range(num_experts):
                    owner, le = divmod(e, epr)
                    cnt = self._view(count_peers[owner], [2, epr], torch.int32)
                    n = int(local_count[e])
                    base[e] = int(cnt[parity, le]) if n > 0 else 0
                    cnt[parity, le] += n
                    local_count[e] = 0
            self._view(count_peers[rank], [2, epr], torch.int32)[parity ^ 1].zero_()
        for i in range(T * k):
            e = int(idx[i])
            if e < 0 or e >= num_experts:
                continue
            owner, le = divmod(e, epr)
            if reuse:
                row = int(slotf[i])
            else:
                r = int(base[e]) + int(posf[i])
                row = le * cap + r if (0 <= r < cap and int(posf[i]) >= 0) else -1
                slotf[i] = row
            if row < 0 or row >= epr * cap:
                self._status(status_addr, 6, 1101)
                continue
            dst = self._view(x_peers[owner], [epr * cap, H], torch.bfloat16)
            src = x[i // k]
            dst[row] = (src.float() * float(row_scale.view(-1)[i])).to(torch.bfloat16) if row_scale is not None else src
            if not reuse:
                self._view(info_peers[owner], [epr * cap], torch.int32)[row] = (rank << 28) | i

    def moe_zero_tail(self, buf, counts, experts_local, cap, width):
        cnt = self._view(counts, [experts_local], torch.int32)
        rows = self._view(buf, [experts_local * cap, width], torch.bfloat16)
        for e in range(experts_local):
            n = min(int(cnt[e]), cap)
            rows[e * cap + n: e * cap + min((n + 127) // 128 * 128, cap)].zero_()

    def moe_combine(self, slots, w, out, topk):
        T, H = out.shape
        v = slots.view(T, topk, H).float()
        out.copy_(((v * w.view(T, topk, 1)) if w is not None else v).sum(1).to(out.dtype))

    def moe_combine_dw(self, dout, slots, dw, topk):
        T, H = dout.shape
        dw.copy_((slots.view(T, topk, H).float() * dout.float().view(T, 1, H)).sum(-1))

    # ---------------------------------------------------------------------------------------- grouped GEMM
    def grouped_gemm(self, mode, G, cap, M, N, K, counts, A, a_mn, lda, gsa, B, b_mn, ldb, gsb, epilogue, out, ldc, gsc,
                     gu, ldgu, dgu, row_info, peers, sgd_lr, zero_tail, group_m, max_ctas, status, peer_rows=0, _fp32_operands=False):
        assert _fp32_operands or (A.dtype == torch.bfloat16 and B.dtype == torch.bfloat16)
        assert A.is_contiguous() and B.is_contiguous()
        assert counts is None or (counts.dtype == torch.int32 and counts.numel() >= G)
        if mode == 1:                                               # K-grouped: C_g = A_g^T @ B_g over the group's rows
            assert epilogue == EPI_WGRAD and A.shape == (G * cap, M) and B.shape == (G * cap, N) and out.shape == (G, M, N)
            for g in range(G):
                n = min(int(counts[g]), cap)
                c = A[g * cap: g * cap + n].float().t() @ B[g * cap: g * cap + n].float()
                out[g] = ((out[g].float() - sgd_lr * c) if sgd_lr else c).to(torch.bfloat16)
            return
        assert A.shape == (G * cap, K) and B.shape[0] == G
        for g in range(G):
            n = min(int(counts[g]), cap) if counts is not None else cap
            tail = min((n + 127) // 128 * 128, cap) if zero_tail else n
            rows = slice(g * cap, g * cap + n)
            pad = slice(g * cap + n, g * cap + tail)
            b = B[g].float()
            c = A[rows].float() @ (b if b_mn else b.t())            # [n, N]
            assert c.shape[1] == N
            if epilogue == EPI_STORE:
                out[rows] = c.to(torch.bfloat16)
                out[pad] = 0
            elif epilogue == EPI_SWIGLU:                            # columns in blocks of 256: 128 gate | 128 up
                v = c.view(n, N // 256, 2, 128)
                gate, up = v[:, :, 0], v[:, :, 1]
                out[rows] = (torch.nn.functional.silu(gate) * up).reshape(n, N // 2).to(torch.bfloat16)
                out[pad] = 0
                if gu is not None:
                    gu[rows] = c.to(torch.bfloat16)
                    gu[pad] = 0
            elif epilogue == EPI_SCATTER:                           # every row goes back to where its token lives
                info = row_info[rows]
                for r in range(n):
                    home, i = (int(info[r]) >> 28) & 0xF, int(info[r]) & 0x0FFFFFFF
                    assert home < len(peers) and (peer_rows <= 0 or i < peer_rows), "the kernel skips such a row and reports a bad index"
                    self._view(peers[home] + i * ldc * 2, [N], torch.bfloat16).copy_(c[r].to(torch.bfloat16))
            elif epilogue == EPI_DSWIGLU:                           # c = dAct [n, F]; saved gate/up -> dGate/dUp, interleaved
                v = gu[rows].float().view(n, N // 128, 2, 128)
                gate, up = v[:, :, 0], v[:, :, 1]
                da = c.view(n, N // 128, 128)
                s = torch.sigmoid(gate)
                dg = da * up * (s * (1 + gate * (1 - s)))
                du = da * gate * s
                dgu[rows] = torch.stack([dg, du], 2).reshape(n, 2 * N).to(torch.bfloat16)
                dgu[pad] = 0
            else:
                raise AssertionError("WGRAD needs the K-grouped mode")


    # ---------------------------------------------------------------------------------------- fp8 arm
    def grouped_gemm_wgrad_push(self, G, cap, counts, A, B, peers, rank, block_log2, group_m, max_ctas, status):
        # dW_g = A_g^T @ B_g, its rows dealt out in blocks to the ranks that sum them: block b of group g lands in rank
        # b % world's staging [G][world sources][M / world][N] at source `rank`
        assert A.dtype == torch.bfloat16 and B.dtype == torch.bfloat16 and A.is_contiguous() and B.is_contiguous()
        M, N, world, blk = A.shape[1], B.shape[1], len(peers), 1 << block_log2
        assert A.shape[0] == G * cap and B.shape[0] == G * cap and M % (world * blk) == 0 and 0 <= rank < world
        own = M // world
        for g in range(G):
            n = min(int(counts[g]), cap)
            c = (A[g * cap: g * cap + n].float().t() @ B[g * cap: g * cap + n].float()).to(torch.bfloat16)
            c = c.view(M // (world * blk), world, blk, N)                    # [round, owner, row in block, N]
            for d in range(world):
                dst = self._view(peers[d] + ((g * world + rank) * own) * N * 2, [own, N], torch.bfloat16)
                dst.copy_(c[:, d].reshape(own, N))

    def shadow_update(self, part, w, out_peers, groups, rank, M, N, block_log2, group_stride, lr, max_ctas):
        world, blk = len(out_peers), 1 << block_log2
        assert part.dtype == torch.bfloat16 and M % (world * blk) == 0 and N % 8 == 0 and group_stride % 8 == 0
        own = M // world
        total = part.reshape(-1)[: groups * M * N].view(groups, world, own, N).float().sum(1)       # [groups, own, N]
        for g in range(groups):
            # local block i, row j -> row (i * world + rank) * blk + j of the full matrix
            rows = ((torch.arange(own // blk).view(-1, 1) * world + rank) * blk + torch.arange(blk).view(1, -1)).reshape(-1)
            new = total[g]
            if lr:
                new = w.reshape(-1)[g * group_stride: g * group_stride + M * N].view(M, N)[rows].float() - lr * new
            new = new.to(torch.bfloat16)
            for d in range(world):
                self._view(out_peers[d] + g * group_stride * 2, [M, N], torch.bfloat16)[rows] = new

    def fp8_quantize_rows(self, x, q, scale, counts, cap):
        from fuselink_b200.ops import fp8 as f8
        rows = x.shape[0]
        live = torch.ones(rows, dtype=torch.bool)
        if counts is not None:                                      # only the rows a group holds are quantised
            live = (torch.arange(rows) % cap) < counts.long().repeat_interleave(cap)[:rows].clamp(max=cap)
        qq, ss = f8.ref_quantize_rows(x[live])
        q[live] = qq
        scale[live] = ss

    def fp8_quantize_blocks(self, w, q, scale):
        from fuselink_b200.ops import fp8 as f8
        G, R, Cc = w.shape
        v = w.float().view(G, R // 128, 128, Cc // 128, 128)
        amax = v.abs().amax((2, 4))
        s = torch.where(amax > 0, amax / f8.FP8_MAX, torch.ones_like(amax))
        q.copy_((v / s.view(G, R // 128, 1, Cc // 128, 1)).clamp(-f8.FP8_MAX, f8.FP8_MAX).to(f8.FP8).view(G, R, Cc))
        scale.copy_(s)

    def fp8_grouped_gemm(self, G, cap, N, K, counts, A, a_scale, B, b_mn, b_scale, epilogue, out, ldc, gu, ldgu, dgu, row_info,
                         peers, zero_tail, group_m, max_ctas, status, peer_rows=0):
        from fuselink_b200.ops import fp8 as f8
        assert A.element_size() == 1 and B.element_size() == 1 and A.shape == (G * cap, K)
        assert a_scale.shape == (G * cap, K // 128)
        assert b_scale.shape == ((G, K // 128, N // 128) if b_mn else (G, N // 128, K // 128)), (b_scale.shape, b_mn, N, K)
        rows = A.shape[0]
        live = torch.ones(rows, dtype=torch.bool)
        if counts is not None:
            live = (torch.arange(rows) % cap) < counts.long().repeat_interleave(cap)[:rows].clamp(max=cap)
        a = torch.zeros(rows, K)
        a[live] = f8.dequantize_rows(A[live], a_scale[live])       # rows beyond a group's count hold stale bytes
        b = f8.dequantize_blocks(B, b_scale)
        # the same epilogues, on operands that carry exactly the information the e4m3 values and their scales hold
        self.grouped_gemm(0, G, cap, 0, N, K, counts, a.to(torch.float32), False, K, cap * K, b, b_mn, 0, 0, epilogue, out, ldc, 0,
                          gu, ldgu, dgu, row_info, peers, 0.0, zero_tail, group_m, max_ctas, status, peer_rows, _fp32_operands=True)


def describe_call(args, bases, span=1 << 30):
    """Arguments of a device call as data: tensors by shape / dtype / contiguity, addresses relative to the heap regions
    they point into, everything else as it is.  Two runs that hand the kernels the same work give the same description."""
    def one(a):
        if torch.is_tensor(a):
            return ["tensor", list(a.shape), str(a.dtype), a.is_contiguous()]
        if isinstance(a, (list, tuple)):
            return ["list", [one(x) for x in a]]
        if isinstance(a, int) and a > (1 << 32):
            for i, b in enumerate(bases):
                if 0 <= a - b < span:
                    return ["addr", i, a - b]
            return ["addr", "outside the heap"]
        return a
    return [one(a) for a in args]


@contextlib.contextmanager
def recording(model, bases, names=("moe_dispatch", "moe_zero_tail", "grouped_gemm", "moe_combine", "moe_combine_dw", "barrier")):
    """Inside the block every call of the named entry points is appended to the list this yields, as [name, description]."""
    trace, cls, saved = [], type(model), {}
    for name in names:
        orig = getattr(cls, name)
        saved[name] = orig

        def wrap(self, *a, _n=name, _o=orig, **k):
            trace.append([_n, describe_call(a, bases)])
            return _o(self, *a, **k)
        setattr(cls, name, wrap)
    try:
        yield trace
    finally:
        for name, orig in saved.items():
            setattr(cls, name, orig)


@contextlib.contextmanager
def installed(single_process=True, lock_path=None):
    """Inside the block the MoE path's and the transfer path's modules get the model instead of the extension.  With
    ``single_process=False`` barriers really wait (the ranks are separate processes over a shared-memory heap)."""
    from fuselink_b200 import _ext
    from fuselink_b200.ops import comm, gemm, moe
    model = Model(_ext.require_native())
    model.single_process = single_process
    model.lock_path = lock_path
    from fuselink_b200.models import dlrm
    from fuselink_b200.ops import fp8
    from fuselink_b200.serving import disagg
    saved = [(m, m.require_native) for m in (comm, gemm, moe, fp8, dlrm, disagg)]
    for m, _ in saved:
        m.require_native = lambda model=model: model
    try:
        yield model
    finally:
        for m, f in saved:
            m.require_native = f
