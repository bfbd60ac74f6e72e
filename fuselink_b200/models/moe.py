"""MoE expert-parallel layer (the workload the reference runs through Megatron-DeepSpeed, .gitmodules:11-13).

``MoELayer`` owns a router and this rank's experts.  On CUDA tensors the forward/backward are the fused
kernels of ``ops/moe.py`` over the symmetric heap; on CPU tensors (multi-process tests over gloo) the same
math runs as plain PyTorch with an all-gather of the tokens and a reduce-scatter of the outputs.
"""
from __future__ import annotations

import dataclasses
import os
from typing import Optional

import torch
import torch.nn as nn

from ..ops import gemm, ref
from ..ops.moe import MoEConfig, MoEFunction, MoEWorkspace, balanced_placement, expert_home
from ..parallel.symm import SymmetricHeap


def zipf_log_bias(num_experts: int, s: float = 1.2) -> torch.Tensor:
    """log of the Zipf(s) pmf over expert ranks 1..E; added to the router logits it skews the load."""
    p = torch.arange(1, num_experts + 1, dtype=torch.float32).pow(-s)
    return (p / p.sum()).log()


def expert_capacity(tokens: int, num_experts: int, topk: int, capacity_factor: float, min_capacity: int = 4) -> int:
    """Rows one expert accepts from one rank's batch: ceil(tokens / experts * factor) per routing choice."""
    import math
    return max(int(math.ceil(tokens / num_experts * capacity_factor)) * topk, min_capacity)


def capacity_keep_mask(idx: torch.Tensor, num_experts: int, capacity: int) -> torch.Tensor:
    """[T, k] bool: which routing choices fit when every expert accepts at most ``capacity`` rows of this batch.
    Choices are admitted in token order, all first choices before any second choice (the GShard / DeepSpeed rule)."""
    T, k = idx.shape
    keep = torch.zeros(T, k, dtype=torch.bool, device=idx.device)
    taken = torch.zeros(num_experts, dtype=torch.long, device=idx.device)
    for j in range(k):
        onehot = torch.nn.functional.one_hot(idx[:, j].long(), num_experts)            # [T, E]
        pos = (onehot.cumsum(0) - 1 + taken.unsqueeze(0)).gather(1, idx[:, j:j + 1].long()).squeeze(1)
        keep[:, j] = pos < capacity
        taken = taken + onehot.sum(0)
    return keep


def load_balancing_loss(probs: torch.Tensor, idx: torch.Tensor, num_experts: int) -> torch.Tensor:
    """E * sum_e (share of tokens whose first choice is e) * (mean router probability of e): 1 when balanced."""
    me = probs.mean(0)
    ce = torch.nn.functional.one_hot(idx[:, 0].long(), num_experts).float().mean(0)
    return (me * ce).sum() * num_experts


class MoELayer(nn.Module):
    """Router + this rank's experts.

    Gating options (what the MoE layer of the reference's Megatron-DeepSpeed experiment exposes): ``capacity_factor``
    with ``drop_tokens`` (choices over an expert's capacity contribute nothing; on the fused path their rows still
    travel, with weight zero, because the transport is sized for the worst case), ``noisy_gate`` ("jitter": inputs of
    the router are scaled by U(1-eps, 1+eps) in training; "rsample": Gumbel noise on the logits), and the
    load-balancing auxiliary loss of the last forward in ``self.l_aux``."""

    def __init__(self, cfg: MoEConfig, heap: Optional[SymmetricHeap] = None, rank: int = 0, world: int = 1,
                 device="cuda", zipf_s: Optional[float] = 1.2, seed: int = 0, fused_sgd_lr: float = 0.0,
                 name: str = "moe", capacity_factor: float = 0.0, drop_tokens: bool = False, min_capacity: int = 4,
                 noisy_gate: Optional[str] = None, jitter_eps: float = 1e-2, shadow_experts=0, placement=None):
        super().__init__()
        bias = zipf_log_bias(cfg.num_experts, zipf_s) if zipf_s else torch.zeros(cfg.num_experts)
        # which rank owns which expert: in order by default; "balanced" evens out the rows per rank the router's bias
        # predicts (the same on every rank, since the bias is); or an explicit tuple of homes
        if placement == "balanced":
            placement = balanced_placement(bias.exp().tolist(), world)
        if placement not in (None, "contiguous") and tuple(placement) != tuple(cfg.placement):
            cfg = dataclasses.replace(cfg, placement=tuple(int(h) for h in placement))
        if isinstance(shadow_experts, int):
            # the n experts the router favours most (its bias is the same on every rank, so is the choice)
            shadow_experts = torch.argsort(bias, descending=True, stable=True)[:shadow_experts].tolist() if shadow_experts > 0 else []
        if tuple(shadow_experts) != tuple(cfg.shadow):
            cfg = dataclasses.replace(cfg, shadow=tuple(int(e) for e in shadow_experts))
        self.cfg, self.rank, self.world = cfg, rank, world
        assert noisy_gate in (None, "jitter", "rsample")
        self.capacity_factor, self.drop_tokens, self.min_capacity = capacity_factor, drop_tokens, min_capacity
        self.noisy_gate, self.jitter_eps = noisy_gate, jitter_eps
        self.l_aux = torch.zeros((), device=device)
        self.dropped_fraction = 0.0
        assert cfg.num_experts % world == 0
        self.epr = cfg.num_experts // world
        self.fused_sgd_lr = fused_sgd_lr
        g = torch.Generator().manual_seed(seed)
        H, F, E = cfg.hidden, cfg.ffn, cfg.num_experts
        self.router = nn.Parameter((torch.randn(E, H, generator=g) * 0.02).to(torch.bfloat16).to(device))
        self.register_buffer("router_bias", bias.to(device))
        # this rank's experts, then its copies of the shadowed experts (ops.moe.slot_table); every expert's init depends on
        # (seed, global expert id), not on the layout, so a copy starts out equal to the owner's expert
        w13, w2 = [], []
        self.local_experts = sorted((e for e in range(E) if self.home(e)[0] == rank), key=lambda e: self.home(e)[1])
        for e in self.local_experts + list(cfg.shadow):
            ge = torch.Generator().manual_seed(seed * 1000 + 17 + max(e, 0))      # e < 0: an empty copy slot, contents unused
            wg = (torch.randn(F, H, generator=ge) * 0.02).to(torch.bfloat16)
            wu = (torch.randn(F, H, generator=ge) * 0.02).to(torch.bfloat16)
            wd = (torch.randn(H, F, generator=ge) * 0.02).to(torch.bfloat16)
            w13.append(gemm.interleave_gate_up(wg, wu))
            w2.append(wd)
        self.w13 = nn.Parameter(torch.stack(w13).to(device))   # [epr + shadows, 2F, H], gate/up interleaved by 128
        self.w2 = nn.Parameter(torch.stack(w2).to(device))     # [epr + shadows, H, F]
        self.ws = MoEWorkspace(heap, cfg, name) if heap is not None else None
        self.register_state_dict_pre_hook(lambda module, prefix, keep_vars: module.weights_ready())
        if (self.ws is not None and world > 1 and len(cfg.shadow) > 0 and os.environ.get("FUSELINK_PUSH_REDUCE", "1") != "0"
                and self.ws.enable_push_reduce(weights=bool(fused_sgd_lr)) and fused_sgd_lr):
            # The copies' gradients are summed by this library (rows pushed from the weight-gradient GEMMs to the rank that
            # sums them; with the fused update the updated rows are written into every copy, so the expert weights live on
            # the symmetric heap).  Without room there, or with FUSELINK_PUSH_REDUCE=0, the sum is an all-reduce.
            for name_, sym in (("w13", self.ws.push.w13), ("w2", self.ws.push.w2)):
                t = sym.local
                t.copy_(getattr(self, name_).detach())
                setattr(self, name_, nn.Parameter(t))
        if self.ws is not None and world > 1 and len(cfg.shadow) > 0 and os.environ.get("FUSELINK_OVERLAP_REDUCE", "0") == "1":
            self._own_reduce_group(world)

    def _own_reduce_group(self, world: int) -> None:
        """Optional (FUSELINK_OVERLAP_REDUCE=1): a NCCL communicator of this layer's own for the sum of the shadow experts'
        gradients, its kernels limited to a few CTAs, so that the sum can run beside the backward GEMMs (which then leave
        those SMs free) instead of after them.  Off by default: measured on 8 B200s with three shadowed experts the
        CTA-limited all-reduce takes longer than the GEMMs it hides behind (19.7 ms per step against 18.7 ms with the
        default communicator after the GEMMs); at 4 GPUs with one shadowed expert the two are equal.  Collective over the
        ranks; on host runs (gloo) an ordinary group is made and only the order of the work changes."""
        try:
            import torch.distributed as dist
            if not (dist.is_available() and dist.is_initialized() and dist.get_world_size() == world):
                return
            if dist.get_backend() == "nccl":
                opts = dist.ProcessGroupNCCL.Options()
                opts.config.max_ctas = self.ws.reduce_ctas
                opts.config.min_ctas = min(8, self.ws.reduce_ctas)
                self.ws.reduce_group = dist.new_group(ranks=list(range(world)), pg_options=opts)
            else:                                    # host runs (gloo): same order of work, an ordinary group
                self.ws.reduce_group = dist.new_group(ranks=list(range(world)))
            self.ws.overlap_reduce = True
        except Exception:  # noqa: BLE001 - an older PyTorch without the option: the default group, no overlap
            self.ws.reduce_group, self.ws.overlap_reduce = None, False

    # -- routing ------------------------------------------------------------------------------------------
    def route(self, x: torch.Tensor):
        xr = x
        if self.training and self.noisy_gate == "jitter":
            xr = x * torch.empty_like(x).uniform_(1.0 - self.jitter_eps, 1.0 + self.jitter_eps)
        logits = (xr @ self.router.t()).float() + self.router_bias
        probs = torch.softmax(logits, dim=-1)
        if self.training and self.noisy_gate == "rsample":
            noisy = logits - torch.log(-torch.log(torch.rand_like(logits).clamp_min(1e-20)))   # Gumbel-max sampling
            _, idx = torch.topk(noisy, self.cfg.topk, dim=-1)
            w = probs.gather(1, idx)
        else:
            w, idx = torch.topk(probs, self.cfg.topk, dim=-1)
        w = w / w.sum(dim=-1, keepdim=True)
        self.last_topk_idx = idx.detach()       # what reshadow() looks at
        self.l_aux = load_balancing_loss(probs, idx, self.cfg.num_experts)
        if self.drop_tokens and self.capacity_factor > 0:
            cap = expert_capacity(x.shape[0], self.cfg.num_experts, self.cfg.topk, self.capacity_factor, self.min_capacity)
            keep = capacity_keep_mask(idx, self.cfg.num_experts, cap)
            self.dropped_fraction = 1.0 - keep.float().mean()
            w = w * keep.to(w.dtype)
        return w, idx.int()

    def home(self, e: int):
        """(owner rank, local index) of expert e."""
        return expert_home(self.cfg.num_experts, self.world, self.cfg.placement, e)

    def weights_ready(self) -> None:
        """Call before reading the expert weights outside a training step (export, comparison, a change of shadows) when
        experts are shadowed and updated by the fused SGD: the rows of this rank's copies are written by the ranks that
        summed them, and this waits, on the current stream, until all of them have.  The next forward pass needs no such
        call.  Collective in the sense that every rank must have finished its step."""
        if self.ws is not None:
            from ..ops.moe import wait_for_copies
            wait_for_copies(self.ws)

    @torch.no_grad()
    def sync_shadow_to_real(self) -> None:
        """Copy this rank's copy of every shadowed expert it owns into the expert's own slot (which receives no rows while
        the expert is shadowed and so goes stale): call before exporting the experts or changing the set of shadows."""
        self.weights_ready()
        for j, e in enumerate(self.cfg.shadow):
            if e >= 0 and self.home(e)[0] == self.rank:
                self.w13[self.home(e)[1]].copy_(self.w13[self.epr + j])
                self.w2[self.home(e)[1]].copy_(self.w2[self.epr + j])

    @torch.no_grad()
    def set_shadows(self, experts, group=None) -> None:
        """Put other experts into the copy slots (the same number of them), between steps: the owners first take back the
        copies they own (they hold the trained weights), then every new shadow's weights go from its owner to the slot on
        every rank.  Collective over the ranks of the layer."""
        experts = tuple(int(e) for e in experts)
        experts = tuple(e for e in experts if e >= 0) + (-1,) * sum(1 for e in experts if e < 0)   # slots in use first
        assert len(experts) <= len(self.cfg.shadow), "more shadows than copy slots"
        assert all(e < self.cfg.num_experts for e in experts) and len({e for e in experts if e >= 0}) == sum(e >= 0 for e in experts), experts
        experts += (-1,) * (len(self.cfg.shadow) - len(experts))
        if experts == tuple(self.cfg.shadow):
            return
        self.sync_shadow_to_real()
        for j, e in enumerate(experts):
            if e < 0:
                continue
            owner, local = self.home(e)
            for w in (self.w13, self.w2):
                slot = w[self.epr + j]
                if owner == self.rank:
                    slot.copy_(w[local])
                if self.world > 1:
                    import torch.distributed as dist
                    dist.broadcast(slot, src=owner if group is None else dist.get_global_rank(group, owner), group=group)
        self.cfg = dataclasses.replace(self.cfg, shadow=experts)
        if self.ws is not None:
            self.ws.set_shadow(experts)

    @torch.no_grad()
    def reshadow(self, topk_idx: Optional[torch.Tensor] = None, group=None, tolerance: Optional[float] = None) -> tuple:
        """Choose the shadows from the routing of a batch (``topk_idx`` of this rank, by default the last one routed; the
        loads are summed over the ranks) and install them; with ``tolerance`` copy slots are left empty (-1) once the busiest rank is within (1 + tolerance) of the
        mean load.  Returns the experts now shadowed.  An optimizer that keeps
        per-parameter state (momentum, Adam moments) keeps the state of a slot, not of the expert that moves into it."""
        from ..ops.moe import choose_shadows
        n = len(self.cfg.shadow)
        if topk_idx is None:
            topk_idx = getattr(self, "last_topk_idx", None)
        if n == 0 or topk_idx is None:
            return tuple(self.cfg.shadow)
        load = torch.bincount(topk_idx.reshape(-1).long().clamp(0, self.cfg.num_experts - 1), minlength=self.cfg.num_experts).double()
        if self.world > 1:
            import torch.distributed as dist
            dist.all_reduce(load, group=group)
        # with a tolerance: only as many copies as it takes to bring the busiest rank within (1 + tolerance) of the mean
        chosen = choose_shadows(load, n) if tolerance is None else choose_shadows(load, n, self.world, tolerance, self.cfg.placement)
        self.set_shadows(chosen, group)
        return chosen

    @torch.no_grad()
    def rebalance(self, topk_idx: Optional[torch.Tensor] = None, group=None, tolerance: float = 0.05) -> tuple:
        """Even out the rows per rank from the routing of a batch (by default the last one routed), between steps:
        replicate as few of the busiest experts as it takes for no rank's OWN experts to exceed (1 + tolerance) x the mean
        load (the other copy slots stay empty), then split the shadowed experts' rows over the ranks' copies so that every
        rank computes about the mean (ops.moe.spread_plan).  Collective over the ranks of the layer.  Returns the experts
        now shadowed."""
        from ..ops.moe import choose_shadows, spread_pattern, spread_plan
        n, E = len(self.cfg.shadow), self.cfg.num_experts
        if topk_idx is None:
            topk_idx = getattr(self, "last_topk_idx", None)
        if n == 0 or topk_idx is None:
            return tuple(self.cfg.shadow)
        mine = torch.bincount(topk_idx.reshape(-1).long().clamp(0, E - 1), minlength=E).double()
        loads = [mine]
        if self.world > 1:
            import torch.distributed as dist
            loads = [torch.empty_like(mine) for _ in range(self.world)]
            dist.all_gather(loads, mine, group=group)
        loads = torch.stack(loads).cpu()
        chosen = choose_shadows(loads.sum(0), n, self.world, tolerance, self.cfg.placement, spread=True)
        self.set_shadows(chosen, group)
        if self.ws is not None:
            plan = spread_plan(loads.tolist(), self.world, chosen, self.cfg.placement)
            self.ws.set_spread(spread_pattern(plan[self.rank], self.cfg.tokens, self.rank))
        return chosen

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        w, idx = self.route(x)
        if x.is_cuda and self.ws is None:
            raise RuntimeError("MoELayer on CUDA needs a SymmetricHeap (the fused kernels write peer memory)")
        if self.ws is not None:          # a heap was given: the fused path (on host memory only in tests that model the kernels)
            return MoEFunction.apply(x, w, idx, self.w13, self.w2, self.ws, self.fused_sgd_lr)
        return self._forward_reference(x, w, idx)

    # -- CPU / gloo path ----------------------------------------------------------------------------------
    def _forward_reference(self, x, w, idx):
        import torch.distributed as dist

        wg, wu = gemm.deinterleave_gate_up(self.w13)
        if self.world == 1:
            return ref.moe_forward(x, idx, w, wg, wu, self.w2).to(x.dtype)
        T = x.shape[0]
        xs = [torch.empty_like(x) for _ in range(self.world)]
        ws_ = [torch.empty_like(w) for _ in range(self.world)]
        ids = [torch.empty_like(idx) for _ in range(self.world)]
        dist.all_gather(xs, x.detach()); dist.all_gather(ws_, w.detach()); dist.all_gather(ids, idx)
        xs[self.rank], ws_[self.rank] = x, w    # keep the autograd edge of the local shard
        xa, wa, ia = torch.cat(xs), torch.cat(ws_), torch.cat(ids)
        homes = torch.tensor(self.cfg.placement or range(self.cfg.num_experts), device=ia.device)[ia.long().clamp(0, self.cfg.num_experts - 1)]
        local = (homes - self.rank * self.epr).to(ia.dtype)
        local = torch.where((local >= 0) & (local < self.epr) & (ia >= 0), local, torch.full_like(local, -1))
        part = ref.moe_forward(xa, local, wa, wg, wu, self.w2)
        parts = list(part.split(T))
        out = torch.empty_like(parts[0])
        dist.reduce_scatter(out, [p.detach().contiguous() for p in parts]) if dist.get_backend() != "gloo" else None
        if dist.get_backend() == "gloo":
            tot = part.detach().clone()
            dist.all_reduce(tot)
            out = tot.split(T)[self.rank]
        return out.to(x.dtype)


def smoke_step(device: str = "cuda:0", tokens: int = 512, hidden: int = 512, ffn: int = 1024) -> float:
    """One tiny forward + backward + update of the MoE layer on one GPU (all experts local)."""
    torch.cuda.set_device(device)
    cfg = MoEConfig(hidden=hidden, ffn=ffn, num_experts=8, topk=2, tokens=tokens)
    heap = SymmetricHeap.create(64 << 20, device=torch.cuda.current_device())
    try:
        layer = MoELayer(cfg, heap, 0, 1, device=device, fused_sgd_lr=0.01)
        x = torch.randn(tokens, hidden, device=device).to(torch.bfloat16).requires_grad_(True)
        out = layer(x)
        loss = out.float().pow(2).mean()
        loss.backward()
        torch.cuda.synchronize()
        heap.check_status("smoke")
        assert x.grad is not None and torch.isfinite(x.grad.float()).all()
        assert layer.router.grad is not None
        return float(loss.detach())
    finally:
        heap.close()
