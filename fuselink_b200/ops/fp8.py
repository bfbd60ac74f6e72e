"""Block-scaled fp8 (e4m3, "1 x 128" scales) arm of the expert GEMMs: quantisation + grouped GEMM entry points
(csrc/kernels/fp8_gemm.cu) and their plain-PyTorch restatements."""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch

from .._ext import require_native
from .gemm import EPI_DSWIGLU, EPI_SCATTER, EPI_STORE, EPI_SWIGLU  # noqa: F401

FP8 = torch.float8_e4m3fn
FP8_MAX = 448.0


def quantize_rows(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """[rows, K] bf16 -> (e4m3 [rows, K], fp32 scales [rows, K/128]); x ~= q * scale per 128-element block."""
    C = require_native()
    rows, K = x.shape
    q = torch.empty(rows, K, dtype=FP8, device=x.device)
    s = torch.empty(rows, K // 128, dtype=torch.float32, device=x.device)
    C.fp8_quantize_rows(x.contiguous(), q, s, None, 0)
    return q, s


def quantize_blocks(w: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """[G, R, C] bf16 -> (e4m3 same shape, fp32 scales [G, R/128, C/128]): one scale per 128 x 128 block."""
    C = require_native()
    G, R, Cc = w.shape
    q = torch.empty(G, R, Cc, dtype=FP8, device=w.device)
    s = torch.empty(G, R // 128, Cc // 128, dtype=torch.float32, device=w.device)
    C.fp8_quantize_blocks(w.contiguous(), q, s)
    return q, s


def grouped_gemm_rows_fp8(a_q: torch.Tensor, a_s: torch.Tensor, b_q: torch.Tensor, b_s: torch.Tensor,
                          counts: Optional[torch.Tensor], cap: int, *, b_mn_major: bool = False, epilogue: int = EPI_STORE,
                          out: Optional[torch.Tensor] = None, gu: Optional[torch.Tensor] = None,
                          dgu: Optional[torch.Tensor] = None, row_info: Optional[torch.Tensor] = None,
                          peers: Optional[List[int]] = None, ldc: Optional[int] = None, zero_tail: bool = False,
                          group_m: int = 16, max_ctas: int = 0, status: Optional[torch.Tensor] = None, peer_rows: int = 0):
    """M-grouped fp8 GEMM: C_g = (A_g * a_s) @ (B_g * b_s)^T with fp32 accumulation.
    b_q: [G, N, K] (K-major) with b_s [G, N/128, K/128]; or with ``b_mn_major`` [G, K, N] with b_s [G, K/128, N/128]."""
    C = require_native()
    G = b_q.shape[0]
    K = a_q.shape[1]
    N = b_q.shape[2] if b_mn_major else b_q.shape[1]
    assert a_q.shape[0] == G * cap
    if epilogue == EPI_STORE and out is None:
        out = torch.empty(G * cap, N, dtype=torch.bfloat16, device=a_q.device)
    if epilogue == EPI_SWIGLU and out is None:
        out = torch.empty(G * cap, N // 2, dtype=torch.bfloat16, device=a_q.device)
    if ldc is None:
        ldc = out.shape[1] if out is not None else N
    C.fp8_grouped_gemm(G, cap, N, K, counts, a_q, a_s, b_q, b_mn_major, b_s, epilogue, out, ldc, gu,
                       gu.shape[1] if gu is not None else 0, dgu, row_info, peers or [], zero_tail, group_m, max_ctas, status, peer_rows)
    return out


# ---- oracles -----------------------------------------------------------------------------------------------------------
def ref_quantize_rows(x: torch.Tensor):
    rows, K = x.shape
    xb = x.float().view(rows, K // 128, 128)
    amax = xb.abs().amax(-1)
    s = torch.where(amax > 0, amax / FP8_MAX, torch.ones_like(amax))
    q = (xb / s.unsqueeze(-1)).clamp(-FP8_MAX, FP8_MAX).to(FP8)
    return q.view(rows, K), s


def dequantize_rows(q: torch.Tensor, s: torch.Tensor) -> torch.Tensor:
    rows, K = q.shape
    return (q.float().view(rows, K // 128, 128) * s.unsqueeze(-1)).view(rows, K)


def dequantize_blocks(q: torch.Tensor, s: torch.Tensor) -> torch.Tensor:
    G, R, Cc = q.shape
    v = q.float().view(G, R // 128, 128, Cc // 128, 128) * s.view(G, R // 128, 1, Cc // 128, 1)
    return v.view(G, R, Cc)
