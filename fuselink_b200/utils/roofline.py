"""Roofline arithmetic against MEASURED peaks of the B200s the numbers were taken on.

The denominators are a plain device copy and a cuBLAS bf16 GEMM measured on the same GPUs (file
``MEASURED_PEAKS.json`` at the repository root when present, otherwise the stated fallback), so a fraction a
little above 1.0 is possible and one far above it means the timed kernel skipped work."""
from __future__ import annotations

import json
import os
from dataclasses import dataclass

_ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

NVLINK_PEER_GBS = 770.0        # measured peer copy per direction over NVLink 5 / NVSwitch (nominal 900)
NVLINK_ALLREDUCE_BUS_GBS = 725.0


@dataclass
class Peaks:
    hbm_gbs: float
    bf16_tflops: float
    bf16_tflops_sustained: float
    source: str


def peaks() -> Peaks:
    path = os.path.join(_ROOT, "MEASURED_PEAKS.json")
    try:
        d = json.load(open(path))
        return Peaks(d["hbm_gbs"], d["bf16_tflops"], d.get("bf16_tflops_sustained", d["bf16_tflops"]), "measured")
    except Exception:
        return Peaks(6650.0, 1590.0, 1400.0, "fallback")


def gemm_fraction(flops: float, ms: float, sustained: bool = False) -> float:
    p = peaks()
    peak = p.bf16_tflops_sustained if sustained else p.bf16_tflops
    return flops / (ms * 1e-3) / 1e12 / peak


def hbm_fraction(nbytes: float, ms: float) -> float:
    return nbytes / (ms * 1e-3) / 1e9 / peaks().hbm_gbs


def fused_target_ms(flops: float, nvlink_bytes: float, sustained: bool = True) -> float:
    """Target time of a fused compute+collective kernel: the slower of its math at the measured GEMM peak and
    its NVLink bytes at the measured per-direction link bandwidth."""
    p = peaks()
    peak = (p.bf16_tflops_sustained if sustained else p.bf16_tflops) * 1e12
    return max(flops / peak, nvlink_bytes / (NVLINK_PEER_GBS * 1e9)) * 1e3


def moe_step_model(tokens_per_gpu: int, world: int, hidden: int, ffn: int, topk: int, rows_on_rank: int, shadows: int = 0) -> dict:
    """FLOPs and NVLink bytes of one MoE fwd+bwd step on the rank that receives `rows_on_rank` routed rows.  ``shadows``
    experts are replicated on every rank: their bf16 weight gradients (3 * hidden * ffn elements each) cross the links in
    one all-reduce per step, 2 (W - 1) / W of the bytes per rank."""
    flops = rows_on_rank * 3 * (2 * hidden * 2 * ffn + 2 * ffn * hidden)
    remote = (world - 1) / world if world > 1 else 0.0
    # per routed row: x in, y out (forward), dy in, dx out (backward); bf16
    nvlink = rows_on_rank * hidden * 2 * 4 * remote + shadows * 3 * hidden * ffn * 2 * 2 * remote
    return {"flops": flops, "nvlink_bytes": nvlink, "target_ms": fused_target_ms(flops, nvlink)}
