"""Python entry points of the tcgen05 grouped GEMM (csrc/kernels/grouped_gemm.cu)."""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from .._ext import require_native

EPI_STORE, EPI_SWIGLU, EPI_SCATTER, EPI_DSWIGLU, EPI_WGRAD = 0, 1, 2, 3, 4


def grouped_gemm_rows(a: torch.Tensor, b: torch.Tensor, counts: Optional[torch.Tensor], cap: int, *,
                      b_mn_major: bool = False, epilogue: int = EPI_STORE, out: Optional[torch.Tensor] = None,
                      gu: Optional[torch.Tensor] = None, dgu: Optional[torch.Tensor] = None,
                      row_info: Optional[torch.Tensor] = None, peers: Optional[List[int]] = None, ldc: Optional[int] = None,
                      zero_tail: bool = False, group_m: int = 16, max_ctas: int = 0,
                      status: Optional[torch.Tensor] = None, peer_rows: int = 0) -> Optional[torch.Tensor]:
    """M-grouped GEMM: for each group g, ``C_g = A_g @ B_g^T`` over the first counts[g] rows of A_g.
    With the SCATTER epilogue ``peer_rows`` is the number of rows of every receive buffer: a row whose return address
    lies outside is not stored and the status word reports a bad index.

    a: [G*cap, K] bf16 token buffer (group g owns rows [g*cap, (g+1)*cap)).
    b: [G, N, K] (K-major, the nn.Linear layout) or, with ``b_mn_major``, [G, K, N].
    """
    C = require_native()
    G = b.shape[0]
    K = a.shape[1]
    N = b.shape[2] if b_mn_major else b.shape[1]
    assert a.shape[0] == G * cap and a.is_contiguous() and b.is_contiguous()
    assert (b.shape[1] if b_mn_major else b.shape[2]) == K
    if epilogue == EPI_STORE and out is None:
        out = torch.empty(G * cap, N, dtype=torch.bfloat16, device=a.device)
    if epilogue == EPI_SWIGLU and out is None:
        out = torch.empty(G * cap, N // 2, dtype=torch.bfloat16, device=a.device)
    if ldc is None:
        ldc = out.shape[1] if out is not None else N
    gsc = cap * ldc
    ldb = N if b_mn_major else K
    C.grouped_gemm(0, G, cap, 0, N, K, counts, a, False, K, cap * K, b, b_mn_major, ldb, b.shape[1] * b.shape[2],
                   epilogue, out, ldc, gsc, gu if gu is not None else None, gu.shape[1] if gu is not None else 0, dgu,
                   row_info, peers or [], 0.0, zero_tail, group_m, max_ctas, status, peer_rows)
    return out


def grouped_gemm_wgrad(a: torch.Tensor, b: torch.Tensor, counts: Optional[torch.Tensor], cap: int, G: int, *,
                       out: Optional[torch.Tensor] = None, sgd_lr: float = 0.0, group_m: int = 16, max_ctas: int = 0,
                       status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """K-grouped GEMM: ``C_g[M, N] = A_g^T @ B_g`` with A_g, B_g the first counts[g] rows of group g in the
    token-major buffers a: [G*cap, M], b: [G*cap, N].  With ``sgd_lr`` the result is applied to ``out`` in place
    (``out -= lr * C``) instead of being stored."""
    C = require_native()
    M, N = a.shape[1], b.shape[1]
    assert a.shape[0] == G * cap and b.shape[0] == G * cap and a.is_contiguous() and b.is_contiguous()
    if out is None:
        assert sgd_lr == 0.0
        out = torch.empty(G, M, N, dtype=torch.bfloat16, device=a.device)
    C.grouped_gemm(1, G, cap, M, N, 0, counts, a, True, M, cap * M, b, True, N, cap * N, EPI_WGRAD, out, N, M * N,
                   None, 0, None, None, [], sgd_lr, False, group_m, max_ctas, status, 0)
    return out


def push_block_log2(M: int, world: int, most: int = 8) -> int:
    """Rows of a pushed weight gradient are dealt out to the ranks in blocks of 2^b rows: the largest b <= ``most`` that
    gives every rank a whole number of blocks, or -1 when M is no multiple of the number of ranks."""
    for b in range(most, -1, -1):
        if M % (world << b) == 0:
            return b
    return -1


def grouped_gemm_wgrad_push(a: torch.Tensor, b: torch.Tensor, counts: torch.Tensor, cap: int, G: int, peers: Sequence[int],
                            rank: int, block_log2: int, *, group_m: int = 16, max_ctas: int = 0,
                            status: Optional[torch.Tensor] = None) -> None:
    """K-grouped GEMM as grouped_gemm_wgrad, but the rows of every ``C_g`` go from the epilogue straight to the ranks
    that sum them: block i (2^block_log2 rows) of group g into ``peers[i % world]``, a buffer laid out
    [G, world, M / world, N], at source ``rank`` and local block ``i // world``.  ``shadow_update`` is the other half."""
    require_native().grouped_gemm_wgrad_push(G, cap, counts, a, b, list(peers), rank, block_log2, group_m, max_ctas, status)


def shadow_update(part: torch.Tensor, w: Optional[torch.Tensor], out_peers: Sequence[int], groups: int, rank: int, M: int,
                  N: int, block_log2: int, group_stride: int, lr: float, max_ctas: int = 0) -> None:
    """For the blocks of rows this rank sums: the fp32 sum over the sources staged in ``part`` ([groups, world, M / world,
    N], written by every rank's grouped_gemm_wgrad_push), then ``w - lr * sum`` (or the sum itself when ``lr`` is 0)
    stored as bf16 into every rank's copy ``out_peers[d]`` ([groups] matrices of [M, N], ``group_stride`` elements
    apart).  Run it once every rank's GEMM is known to be complete."""
    require_native().shadow_update(part, w, list(out_peers), groups, rank, M, N, block_log2, group_stride, lr, max_ctas)


def interleave_gate_up(w_gate: torch.Tensor, w_up: torch.Tensor, block: int = 128) -> torch.Tensor:
    """[.., F, H] gate and up projections -> [.., 2F, H] with rows in blocks [128 gate | 128 up], the layout
    the SWIGLU epilogue expects (one 256-wide accumulator tile holds matching gate and up columns)."""
    *lead, F, H = w_gate.shape
    assert F % block == 0
    g = w_gate.reshape(*lead, F // block, 1, block, H)
    u = w_up.reshape(*lead, F // block, 1, block, H)
    return torch.cat([g, u], dim=-3).reshape(*lead, 2 * F, H).contiguous()


def deinterleave_gate_up(w13: torch.Tensor, block: int = 128):
    *lead, F2, H = w13.shape
    v = w13.reshape(*lead, F2 // (2 * block), 2, block, H)
    return v[..., 0, :, :].reshape(*lead, F2 // 2, H), v[..., 1, :, :].reshape(*lead, F2 // 2, H)
