"""The stock formulation of the MoE expert-parallel step, used as the measured baseline:
framework permute (sort by expert) + ``all_to_all_single`` over NCCL + library GEMMs per expert + the mirror
all-to-all, with autograd doing the backward and ``torch.optim.SGD`` the update.  None of this library's
kernels run on this path.

The expert FFN is the library's grouped GEMM (``torch.nn.functional.grouped_mm``: one launch per projection over all
local experts, group sizes read on the device) where this PyTorch build has it for the device, else one matmul per
expert; the activation stays in bf16.  ``self.expert_gemm`` says which one runs.  The host reads the routing result only
where the stock collective needs it: ``all_to_all_single`` takes its split sizes as Python lists."""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops.moe import MoEConfig
from .moe import zipf_log_bias


class BaselineMoELayer(nn.Module):
    def __init__(self, cfg: MoEConfig, rank: int = 0, world: int = 1, device="cuda", zipf_s=1.2, seed: int = 0, placement=None):
        super().__init__()
        self.cfg, self.rank, self.world = cfg, rank, world
        self.epr = cfg.num_experts // world
        # which rank owns which expert: in order, or "balanced" by the router's bias like MoELayer (ops.moe.balanced_placement)
        homes = list(range(cfg.num_experts))
        if placement == "balanced":
            from ..ops.moe import balanced_placement
            homes = list(balanced_placement((zipf_log_bias(cfg.num_experts, zipf_s) if zipf_s else torch.zeros(cfg.num_experts)).exp().tolist(), world))
        elif placement not in (None, "contiguous"):
            homes = [int(h) for h in placement]
        self.homes = None if homes == list(range(cfg.num_experts)) else torch.tensor(homes, device=device)
        local = sorted((e for e in range(cfg.num_experts) if homes[e] // self.epr == rank), key=lambda e: homes[e])
        g = torch.Generator().manual_seed(seed)
        H, Fd, E = cfg.hidden, cfg.ffn, cfg.num_experts
        self.router = nn.Parameter((torch.randn(E, H, generator=g) * 0.02).to(torch.bfloat16).to(device))
        bias = zipf_log_bias(E, zipf_s) if zipf_s else torch.zeros(E)
        self.register_buffer("router_bias", bias.to(device))
        w13, w2 = [], []
        for e in local:                                            # rank * epr + le in the in-order placement
            ge = torch.Generator().manual_seed(seed * 1000 + 17 + e)
            wg = (torch.randn(Fd, H, generator=ge) * 0.02).to(torch.bfloat16)
            wu = (torch.randn(Fd, H, generator=ge) * 0.02).to(torch.bfloat16)
            wd = (torch.randn(H, Fd, generator=ge) * 0.02).to(torch.bfloat16)
            w13.append(torch.cat([wg, wu], 0))
            w2.append(wd)
        self.w13 = nn.Parameter(torch.stack(w13).to(device))
        self.w2 = nn.Parameter(torch.stack(w2).to(device))
        self.expert_gemm = "grouped_mm" if self._probe_grouped_mm(device) else "matmul per expert"

    @staticmethod
    def _probe_grouped_mm(device) -> bool:
        """Whether the library grouped GEMM runs (forward and backward) on this device with bf16 operands."""
        fn = getattr(F, "grouped_mm", None)
        if fn is None or torch.device(device).type != "cuda":
            return False
        try:
            a = torch.randn(32, 64, device=device, dtype=torch.bfloat16, requires_grad=True)
            b = torch.randn(2, 64, 32, device=device, dtype=torch.bfloat16, requires_grad=True)
            offs = torch.tensor([16, 32], device=device, dtype=torch.int32)
            fn(a, b, offs=offs).float().sum().backward()
            torch.cuda.synchronize()
            return bool(torch.isfinite(a.grad.float()).all())
        except Exception:  # noqa: BLE001 - not supported by this build / device: use the loop
            return False

    def _experts(self, xe, ecnt_dev, ecnt_host):
        """SwiGLU FFN of every local expert over its rows (xe is sorted by expert; ecnt = rows per expert)."""
        Fd = self.cfg.ffn
        if self.expert_gemm == "grouped_mm":
            offs = ecnt_dev.cumsum(0).to(torch.int32)
            h = F.grouped_mm(xe, self.w13.transpose(1, 2), offs=offs)
            return F.grouped_mm(F.silu(h[:, :Fd]) * h[:, Fd:], self.w2.transpose(1, 2), offs=offs)
        ecnt = ecnt_host() if callable(ecnt_host) else ecnt_host
        outs, o = [], 0
        for e in range(self.epr):
            xs = xe[o:o + ecnt[e]]
            o += ecnt[e]
            h = xs @ self.w13[e].t()
            outs.append((F.silu(h[:, :Fd]) * h[:, Fd:]) @ self.w2[e].t())
        return torch.cat(outs)

    def forward(self, x):
        cfg, W = self.cfg, self.world
        T, k, E = x.shape[0], cfg.topk, cfg.num_experts
        logits = (x @ self.router.t()).float() + self.router_bias
        probs = torch.softmax(logits, -1)
        w, idx = torch.topk(probs, k, -1)
        w = w / w.sum(-1, keepdim=True)
        flat = idx.reshape(-1)
        if self.homes is not None:
            flat = self.homes[flat]                                # from here on "expert" means the expert's home slot
        order = torch.argsort(flat, stable=True)
        tok = order // k
        xp = x[tok]                                                # permute
        cnt = torch.bincount(flat, minlength=E)
        if W > 1:
            import torch.distributed as dist
            from torch.distributed.nn.functional import all_to_all_single

            recv_cnt = torch.empty_like(cnt)
            dist.all_to_all_single(recv_cnt, cnt)                  # [W, epr] counts from every rank
            send_sizes = cnt.view(W, self.epr).sum(1).tolist()
            recv_sizes = recv_cnt.view(W, self.epr).sum(1).tolist()
            xr = all_to_all_single(torch.empty(sum(recv_sizes), x.shape[1], dtype=x.dtype, device=x.device), xp,
                                   recv_sizes, send_sizes)
            # received rows are grouped (src rank, local expert): regroup by expert
            rc = recv_cnt.view(W, self.epr)
            eid = torch.repeat_interleave(torch.arange(self.epr, device=x.device).repeat(W), rc.reshape(-1))
            eorder = torch.argsort(eid, stable=True)
            xe = xr[eorder]
            ecnt_dev = rc.sum(0)
        else:
            xe, ecnt_dev = xp, cnt
        ye = self._experts(xe, ecnt_dev, ecnt_dev.tolist)
        if W > 1:
            inv = torch.empty_like(eorder)
            inv[eorder] = torch.arange(eorder.numel(), device=x.device)
            yr = ye[inv]
            yp = all_to_all_single(torch.empty_like(xp), yr, send_sizes, recv_sizes)
        else:
            yp = ye
        wflat = w.reshape(-1)[order].to(yp.dtype).unsqueeze(1)
        out = torch.zeros_like(x).index_add_(0, tok, yp * wflat)   # un-permute + weighted combine
        return out
