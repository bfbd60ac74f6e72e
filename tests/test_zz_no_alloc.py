"""The allocation-free MoE dispatch entry point, called through its exported C symbol.

Some embedders of the library may not allocate device memory where they call it (a communication library's
progress thread, a plugin inside a process whose allocator owns the whole GPU, a latency-bounded serving
loop), so `fl_moe_dispatch_noalloc` keeps its scratch in a fixed array inside the library.  The test calls
it twice in a row through ctypes and compares what it produced with what the regular entry point (scratch
passed in by the caller) produces for the same routing.
"""
import ctypes
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


class Args(ctypes.Structure):
    _fields_ = [
        ("x", ctypes.c_void_p), ("topk_idx", ctypes.c_void_p), ("row_scale", ctypes.c_void_p),
        ("tokens", ctypes.c_int), ("topk", ctypes.c_int), ("hidden", ctypes.c_int),
        ("num_experts", ctypes.c_int), ("experts_per_rank", ctypes.c_int), ("cap", ctypes.c_int),
        ("rank", ctypes.c_int), ("world", ctypes.c_int),
        ("slot", ctypes.c_void_p),
        ("count_peers", ctypes.c_void_p * 8), ("parity", ctypes.c_int),
        ("x_peers", ctypes.c_void_p * 8), ("info_peers", ctypes.c_void_p * 8),
        ("status", ctypes.c_void_p),
    ]


def _lib():
    import fuselink_b200
    path = os.path.join(os.path.dirname(fuselink_b200.__file__), "_C.so")
    lib = ctypes.CDLL(path)
    lib.fl_moe_dispatch_noalloc.argtypes = [ctypes.POINTER(Args), ctypes.c_void_p]
    lib.fl_moe_dispatch_noalloc.restype = ctypes.c_int
    lib.fl_moe_dispatch_noalloc_error.restype = ctypes.c_char_p
    lib.fl_moe_dispatch_noalloc_setup.restype = ctypes.c_int
    return lib


def _buffers(E, cap, H):
    return (torch.zeros(E * cap, H, dtype=torch.bfloat16, device="cuda"),
            torch.full((E * cap,), -1, dtype=torch.int32, device="cuda"),
            torch.zeros(2, E, dtype=torch.int32, device="cuda"))


def test_noalloc_dispatch_matches_regular_entry_point():
    from fuselink_b200 import C
    lib = _lib()
    T, k, H, E = 1000, 2, 256, 8
    cap = 1024
    stream = torch.cuda.current_stream().cuda_stream
    assert lib.fl_moe_dispatch_noalloc_setup() == 0, lib.fl_moe_dispatch_noalloc_error()
    for call in range(2):                       # two calls in a row share the built-in scratch
        g = torch.Generator(device="cuda").manual_seed(7 + call)
        x = torch.randn(T, H, generator=g, device="cuda").to(torch.bfloat16)
        idx = torch.stack([torch.randperm(E, generator=g, device="cuda")[:k] for _ in range(T)]).int().contiguous()
        parity = call & 1
        # regular entry point: the caller provides the scratch
        xd_a, info_a, cnt_a = _buffers(E, cap, H)
        slot_a = torch.zeros(T, k, dtype=torch.int32, device="cuda")
        lc = torch.zeros(E, dtype=torch.int32, device="cuda")
        base = torch.zeros(E, dtype=torch.int32, device="cuda")
        pos = torch.zeros(T, k, dtype=torch.int32, device="cuda")
        C.moe_dispatch(x, idx, None, E, E, cap, 0, 1, lc, base, pos, slot_a, [cnt_a.data_ptr()], parity,
                       [xd_a.data_ptr()], [info_a.data_ptr()], False, 0)
        # allocation-free entry point through the C symbol
        xd_b, info_b, cnt_b = _buffers(E, cap, H)
        slot_b = torch.zeros(T, k, dtype=torch.int32, device="cuda")
        status = torch.zeros(8, dtype=torch.int32, device="cuda")
        a = Args()
        a.x, a.topk_idx, a.row_scale = x.data_ptr(), idx.data_ptr(), None
        a.tokens, a.topk, a.hidden = T, k, H
        a.num_experts, a.experts_per_rank, a.cap, a.rank, a.world = E, E, cap, 0, 1
        a.slot = slot_b.data_ptr()
        a.count_peers[0], a.x_peers[0], a.info_peers[0] = cnt_b.data_ptr(), xd_b.data_ptr(), info_b.data_ptr()
        a.parity = parity
        a.status = status.data_ptr()
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        rc = lib.fl_moe_dispatch_noalloc(ctypes.byref(a), ctypes.c_void_p(stream))
        assert rc == 0, lib.fl_moe_dispatch_noalloc_error()
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == free_before, "the call must not change the device's free memory"
        assert status[0].item() == 0
        # same per-expert counts; every (token, k) row landed intact in its expert's range; same return info
        assert torch.equal(cnt_a[parity], cnt_b[parity])
        assert torch.equal(cnt_b[parity].cpu(), torch.bincount(idx.reshape(-1).cpu().long(), minlength=E).int())
        sa, sb = slot_a.reshape(-1).long(), slot_b.reshape(-1).long()
        assert torch.equal(sa // cap, sb // cap), "rows must land in the same expert's buffer"
        assert sb.unique().numel() == T * k, "every assignment needs its own row"
        assert torch.equal(xd_a[sa], xd_b[sb])
        assert torch.equal(xd_b[sb], x.repeat_interleave(k, 0))
        assert torch.equal(info_a[sa], info_b[sb])
        assert torch.equal(info_b[sb].cpu(), torch.arange(T * k, dtype=torch.int32))


def test_noalloc_dispatch_rejects_oversized_problem():
    lib = _lib()
    a = Args()
    a.tokens, a.topk, a.hidden = 128 * 1024, 2, 256          # tokens * topk beyond the built-in scratch
    a.num_experts, a.experts_per_rank, a.cap, a.rank, a.world = 8, 8, 1024, 0, 1
    rc = lib.fl_moe_dispatch_noalloc(ctypes.byref(a), None)
    assert rc == -100
    assert b"too large" in lib.fl_moe_dispatch_noalloc_error()
    a.tokens, a.rank = 64, 3                                  # a rank outside the world: refused before anything is enqueued
    assert lib.fl_moe_dispatch_noalloc(ctypes.byref(a), None) == -102
    assert b"rank" in lib.fl_moe_dispatch_noalloc_error()
