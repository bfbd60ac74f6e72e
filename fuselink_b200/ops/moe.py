"""Expert-parallel MoE forward/backward built from the fused kernels.

Per step and rank (E experts over W ranks, top-k routing, SwiGLU experts):

forward   dispatch (permute + scatter into the expert owners' buffers over NVLink)  -> flag barrier ->
          GEMM1 (tcgen05, SWIGLU epilogue) -> GEMM2 (tcgen05, SCATTER epilogue: rows return to the token's home
          rank inside the GEMM) -> flag barrier -> weighted combine
backward  dw = <dOut, y_k>; dispatch(w_k * dOut) to the slots chosen in forward -> barrier ->
          dAct GEMM (B MN-major, DSWIGLU epilogue) -> wgrad W2, wgrad W13 (K-grouped, both operands MN-major)
          -> dX GEMM (B MN-major, SCATTER epilogue) -> barrier -> sum over k

There is no stand-alone all-to-all and no framework permute in either direction, and NCCL is not called.  When experts
are shadowed (``MoEConfig.shadow``, ``slot_table``) a hot expert is replicated on every rank, its rows are computed on any
rank's copy, and the copies' weight gradients are summed over the ranks by two more kernels of this library
(``MoEWorkspace.enable_push_reduce``: the weight-gradient GEMM's epilogue stores each block of result rows into the
staging of the rank that sums it; that rank writes the updated rows, or the summed gradient rows, into every copy).
Where that is not possible (rows that do not divide over the ranks, no room on the heap, FUSELINK_PUSH_REDUCE=0) the sum
is one all-reduce per step on the process group.
"""
from __future__ import annotations

import dataclasses
import types
from dataclasses import dataclass
from typing import Optional, Sequence, Tuple

import torch

from .._ext import require_native
from ..parallel.symm import SymmetricHeap
from . import gemm
from .comm import barrier


@dataclass
class MoEConfig:
    hidden: int = 4096
    ffn: int = 14336
    num_experts: int = 8
    topk: int = 2
    tokens: int = 8192          # tokens per rank and step
    fp8: bool = False           # block-scaled e4m3 ("1 x 128") for the forward and dgrad GEMMs; wgrad stays bf16
    placement: Tuple[int, ...] = ()  # home of every expert as rank * (E / W) + local index; () = in order (expert e on rank
                                     # e // (E / W)); see balanced_placement()
    shadow: Tuple[int, ...] = ()  # experts replicated on every rank ("shadow" experts), see slot_table(); one entry per copy
                                  # slot, the slots in use first, -1 for a slot that is empty at the moment


def balanced_placement(expected_load: Sequence[float], world: int) -> Tuple[int, ...]:
    """Homes for the experts that even out the expected rows per rank: experts in order of decreasing load, each to the
    rank that carries the least so far and still has a free place (longest-processing-time-first).  With one expert per
    rank, or one rank, this is the in-order placement.  Returns home[e] = rank * (E / W) + local index."""
    E = len(expected_load)
    assert E % world == 0
    real = E // world
    if real == 1 or world == 1:
        return tuple(range(E))
    load, used, home = [0.0] * world, [0] * world, [0] * E
    for e in sorted(range(E), key=lambda e: (-float(expected_load[e]), e)):
        r = min((r for r in range(world) if used[r] < real), key=lambda r: (load[r], r))
        home[e] = r * real + used[r]
        used[r] += 1
        load[r] += float(expected_load[e])
    return tuple(home)


def expert_home(num_experts: int, world: int, placement: Sequence[int], e: int) -> Tuple[int, int]:
    """(owner rank, local index) of expert e."""
    h = placement[e] if placement else e
    return divmod(h, num_experts // world)


def slot_table(num_experts: int, world: int, shadow: Sequence[int], rank: int, placement: Sequence[int] = ()) -> torch.Tensor:
    """Where rank ``rank`` sends a row that chose expert e: the slot number ``dest_rank * slots_per_rank + local_slot``.

    Every rank has ``E / W`` slots for the experts it owns followed by one slot per shadowed expert.  A row for an
    ordinary expert goes to the owner's slot (``placement`` says who owns what; in order by default).  A row for a
    shadowed expert stays on the rank it comes from, in that rank's copy of the expert; the owner's own slot for it stays
    empty.  This is what removes the load imbalance of a skewed router: a hot expert's rows are computed where they
    originate, spread over all ranks, at the price of summing that expert's weight gradients over the ranks (FasterMoE
    calls such replicas shadow experts).  The kernels see slots as "experts" and need no change:
    owner = slot // slots_per_rank.

    The table has E + 2 entries and is indexed with ``clamp(e, -1, E) + 1``, so an expert id out of range maps to -1,
    which the dispatch kernel reports through the status word like any other bad index."""
    assert num_experts % world == 0
    real = num_experts // world
    spr = real + len(shadow)
    used = [e for e in shadow if e >= 0]
    assert len(set(used)) == len(used) and all(e < num_experts for e in used)
    assert list(shadow[:len(used)]) == used, "the copy slots in use come first"
    assert not placement or sorted(placement) == list(range(num_experts)), "a placement gives every expert a home of its own"
    t = torch.full((num_experts + 2,), -1, dtype=torch.int32)
    for e in range(num_experts):
        owner, local = expert_home(num_experts, world, placement, e)
        t[e + 1] = owner * spr + local
    for j, e in enumerate(used):
        t[e + 1] = rank * spr + real + j
    return t


class MoEWorkspace:
    """Symmetric and local buffers of one MoE layer on one rank.  Sized for the worst case: every token of
    every rank may choose the same expert, so each expert buffer holds tokens*world rows."""

    def __init__(self, heap: SymmetricHeap, cfg: MoEConfig, name: str = "moe"):
        self.heap, self.cfg, self.name = heap, cfg, name
        W = heap.world
        assert cfg.num_experts % W == 0, "experts must divide evenly over ranks"
        self.epr_real = cfg.num_experts // W              # experts this rank owns
        self.nshadow = len(cfg.shadow)                    # + its copy slots for shadowed experts (some may be empty)
        self.epr = self.epr_real + self.nshadow           # slots per rank: what the kernels call experts per rank
        self.num_slots = W * self.epr
        assert self.epr <= 64, "the grouped GEMM takes at most 64 groups per launch"
        self.cap = (cfg.tokens * W + 127) // 128 * 128
        rows = self.epr * self.cap
        H, F, T, k = cfg.hidden, cfg.ffn, cfg.tokens, cfg.topk
        bf = torch.bfloat16
        # symmetric (peers write into these)
        self.xd = heap.alloc_tensor([rows, H], bf)        # dispatched tokens
        self.dyd = heap.alloc_tensor([rows, H], bf)       # dispatched output gradients
        self.info = heap.alloc_tensor([rows], torch.int32)
        self.counts = heap.alloc_tensor([2, self.epr], torch.int32)
        self.comb = heap.alloc_tensor([T * k, H], bf)     # expert outputs y_k returned to the home rank
        self.dxs = heap.alloc_tensor([T * k, H], bf)      # input gradients returned to the home rank
        dev = self.xd.local.device
        # local
        self.act = torch.empty(rows, F, dtype=bf, device=dev)
        self.gu = torch.empty(rows, 2 * F, dtype=bf, device=dev)
        self.dgu = torch.empty(rows, 2 * F, dtype=bf, device=dev)
        self.local_count = torch.zeros(self.num_slots + 1, dtype=torch.int32, device=dev)   # + the ticket of the one-launch count/reserve
        self.base = torch.zeros(self.num_slots, dtype=torch.int32, device=dev)
        remap = self.nshadow or (cfg.placement and tuple(cfg.placement) != tuple(range(cfg.num_experts)))
        self.slots_of = slot_table(cfg.num_experts, W, cfg.shadow, heap.rank, cfg.placement).to(dev) if remap else None
        self.spread = None                                # [T, 1] int32: rank that computes a token's shadow rows, minus this rank
        self.sh_stride = self._shadow_stride() if self.nshadow else None
        # sums the shadow experts' weight gradients over the ranks, in place; replaced in tests that emulate ranks on one GPU
        self.reduce_shadow_grads = _allreduce_shadow_grads
        self.pos = torch.zeros(T, k, dtype=torch.int32, device=dev)
        self.slot = torch.zeros(T, k, dtype=torch.int32, device=dev)
        if cfg.fp8:
            from . import fp8 as _f8
            f8 = _f8.FP8
            self.q_in = torch.empty(rows, H, dtype=f8, device=dev)          # quantised xd / dyd
            self.s_in = torch.empty(rows, H // 128, dtype=torch.float32, device=dev)
            self.q_act = torch.empty(rows, F, dtype=f8, device=dev)         # quantised act
            self.s_act = torch.empty(rows, F // 128, dtype=torch.float32, device=dev)
            self.q_dgu = torch.empty(rows, 2 * F, dtype=f8, device=dev)     # quantised dgate/dup
            self.s_dgu = torch.empty(rows, 2 * F // 128, dtype=torch.float32, device=dev)
            self.wq = {}                                                     # per-weight (e4m3, scales), refreshed each step
        self.pending_shadow = None
        # Sum of the copies' weight gradients done by this library instead of an all-reduce (enable_push_reduce): the
        # copies' weight-gradient GEMMs store their result rows into the staging of the rank that sums them, and that rank
        # writes the updated rows into every copy.
        self.push = None
        self.gathering_shadow = None
        self.copies_pending = False
        # Overlap of the shadow experts' gradient all-reduce with the rest of the backward pass (set by MoELayer once it has
        # a communicator of its own whose kernels are limited to `reduce_ctas` CTAs): the copies' weight gradients are then
        # computed first and summed while dX and the owned experts' weight gradients run on the remaining SMs.
        self.overlap_reduce = False
        self.reduce_group = None
        self.reduce_ctas = 16
        self.started_shadow = None
        self.parity = 0
        self.step_parity = 0
        self.launches = 0   # kernels of this library launched through this workspace (bench accounting)

    def enable_push_reduce(self, weights: bool = True, max_ctas: int = 0) -> bool:
        """Moves the sum of the shadow experts' weight gradients from an all-reduce into this library's kernels.  Allocates,
        on the symmetric heap, the staging the partial gradients are pushed into and, with ``weights`` (the fused SGD
        update), the expert weights themselves (``self.push.w13`` / ``.w2``: the layer must use these as its parameters,
        since peers write the updated rows of the copies into them); without ``weights`` the buffers the summed gradients
        of the copies are written into by the ranks that sum them (``self.push.g13`` / ``.g2``).  Returns False, and changes
        nothing that matters, when the shapes do not divide over the ranks or the heap has no room; call it on every rank
        or on none."""
        cfg, W = self.cfg, self.heap.world
        H, F = cfg.hidden, cfg.ffn
        b13, b2 = gemm.push_block_log2(2 * F, W), gemm.push_block_log2(H, W)
        if W < 2 or not self.nshadow or b13 < 0 or b2 < 0 or H % 8 or F % 8:
            return False
        try:
            bf = torch.bfloat16
            w13 = self.heap.alloc_tensor([self.epr, 2 * F, H], bf) if weights else None
            w2 = self.heap.alloc_tensor([self.epr, H, F], bf) if weights else None
            g13 = None if weights else self.heap.alloc_tensor([self.nshadow, 2 * F, H], bf)
            g2 = None if weights else self.heap.alloc_tensor([self.nshadow, H, F], bf)
            p13 = self.heap.alloc_tensor([self.nshadow, W, 2 * F // W, H], bf)
            p2 = self.heap.alloc_tensor([self.nshadow, W, H // W, F], bf)
        except MemoryError:
            return False
        self.push = types.SimpleNamespace(w13=w13, w2=w2, g13=g13, g2=g2, p13=p13, p2=p2, b13=b13, b2=b2, max_ctas=max_ctas)
        return True

    def counts_now(self) -> torch.Tensor:
        return self.counts.local[self.step_parity]

    @property
    def shadows_in_use(self) -> int:
        return sum(1 for e in self.cfg.shadow if e >= 0)

    def _shadow_stride(self) -> torch.Tensor:
        """[E + 2] int32, indexed like slots_of: slots per rank for a shadowed expert, 0 for every other entry, so that
        slots_of[j] + sh_stride[j] * (dest - rank) is the expert's copy on rank ``dest``."""
        t = torch.zeros(self.cfg.num_experts + 2, dtype=torch.int32)
        for e in self.cfg.shadow:
            if e >= 0:
                t[e + 1] = self.epr
        return t.to(self.local_count.device)

    def set_spread(self, pattern: Optional[torch.Tensor]) -> None:
        """Which rank computes the shadow rows of each token (spread_pattern), or None: they stay here.  Between steps
        only: the backward dispatch must see the pattern of its forward."""
        assert self.pending_shadow is None
        if pattern is None or not self.nshadow or not bool((pattern != 0).any()):
            self.spread = None
        else:
            assert pattern.numel() == self.cfg.tokens
            self.spread = pattern.to(self.local_count.device, torch.int32).reshape(-1, 1)

    def set_shadow(self, shadow: Sequence[int]) -> None:
        """Other experts in the copy slots (as many slots as before: the buffers keep their size; -1 = empty, in-use slots
        first).  Between steps only."""
        assert len(shadow) == self.nshadow and self.pending_shadow is None
        self.cfg = dataclasses.replace(self.cfg, shadow=tuple(int(e) for e in shadow))
        if self.nshadow:
            self.slots_of = slot_table(self.cfg.num_experts, self.heap.world, self.cfg.shadow, self.heap.rank, self.cfg.placement).to(self.slots_of.device)
            self.sh_stride = self._shadow_stride()
            self.spread = None                            # a plan belongs to the set of shadows it was made for


def owned_rows(expert_load: Sequence[float], world: int, shadow: Sequence[int], placement: Sequence[int] = ()) -> list:
    """Rows every rank computes for the experts it owns that are not shadowed."""
    E = len(expert_load)
    sh = {e for e in shadow if e >= 0}
    per_rank = [0.0] * world
    for e in range(E):
        if e not in sh:
            per_rank[expert_home(E, world, placement, e)[0]] += expert_load[e]
    return per_rank


def busiest_rank_load(expert_load: Sequence[float], world: int, shadow: Sequence[int], placement: Sequence[int] = (),
                      spread: bool = False) -> float:
    """Rows on the busiest rank when the experts in ``shadow`` are replicated: a rank computes the rows of the experts it
    owns that are not shadowed, plus its own share (taken as 1 / world) of every shadowed expert's rows.  With ``spread``
    the shadowed experts' rows go to whichever copies even out the ranks (spread_plan), so the busiest rank carries the
    mean unless the experts it owns alone exceed it."""
    per_rank = owned_rows(expert_load, world, shadow, placement)
    if spread:
        return max(max(per_rank), sum(expert_load) / world)
    return max(per_rank) + sum(expert_load[e] for e in {e for e in shadow if e >= 0}) / world


def spread_plan(load, world: int, shadow: Sequence[int], placement: Sequence[int] = ()) -> list:
    """Where the rows of the shadowed experts are computed so that every rank ends up with the same number of rows.

    ``load[r][e]`` = rows rank r routes to expert e.  Every rank holds a copy of every shadowed expert, so a row for one of
    them may be computed anywhere; by default it stays where it originates.  That leaves the ranks that also own a busy
    ordinary expert with more rows than the others.  The plan moves the surplus: a rank whose total (rows of its own experts
    from everyone + its own shadow rows) is above the mean sends the excess shadow rows to the ranks below the mean, in
    proportion to their deficit.  Returns share[r][d] = fraction of rank r's shadow rows that are computed on rank d (each row
    sums to 1).  The gradients of the copies are summed over the ranks whatever the split, so only the dispatch changes."""
    E = len(load[0])
    sh = [e for e in shadow if e >= 0]
    total = [sum(load[r][e] for r in range(world)) for e in range(E)]
    own = owned_rows(total, world, sh, placement)
    made = [sum(load[r][e] for e in sh) for r in range(world)]          # shadow rows that originate on rank r
    share = [[1.0 if d == r else 0.0 for d in range(world)] for r in range(world)]
    if not sh or sum(made) <= 0:
        return share
    mean = sum(total) / world
    have = [own[r] + made[r] for r in range(world)]
    surplus = [min(max(have[r] - mean, 0.0), made[r]) for r in range(world)]   # only shadow rows can move
    deficit = [max(mean - have[r], 0.0) for r in range(world)]
    moved = min(sum(surplus), sum(deficit))
    if moved <= 0:
        return share
    fs, fd = moved / sum(surplus), moved / sum(deficit)
    for r in range(world):
        out = surplus[r] * fs
        if out <= 0 or made[r] <= 0:
            continue
        share[r][r] = 1.0 - out / made[r]
        for d in range(world):
            if deficit[d] > 0:
                share[r][d] += (out / made[r]) * (deficit[d] * fd / moved)
    return share


def spread_pattern(share_row: Sequence[float], tokens: int, rank: int) -> torch.Tensor:
    """int32 [tokens]: the rank that computes the shadow rows of token t, minus ``rank`` (0 = stays here), such that the
    fraction of tokens sent to rank d is share_row[d].  Token t is placed by the fractional part of t x the golden ratio, a
    low-discrepancy sequence, so every stretch of the batch is split in the same proportions."""
    edges = torch.tensor(list(share_row), dtype=torch.float64).cumsum(0)
    edges = edges / edges[-1]
    u = (torch.arange(tokens, dtype=torch.float64) * 0.6180339887498949) % 1.0
    dest = torch.bucketize(u, edges[:-1].contiguous(), right=True)
    return (dest - rank).to(torch.int32)


def choose_shadows(expert_load: torch.Tensor, slots: int, world: int = 0, tolerance: float = 0.0,
                   placement: Sequence[int] = (), spread: bool = False) -> Tuple[int, ...]:
    """Which experts to replicate, from the rows routed to each expert summed over all ranks: the busiest experts first
    (ties: the lower id), one per copy slot.  With ``world`` and ``tolerance`` given, experts are added only while the
    busiest rank would still carry more than (1 + tolerance) x the mean, so a router that has become balanced stops paying
    for gradient all-reduces; the slots left over are returned as -1."""
    load = [float(v) for v in expert_load.double().cpu()]
    order = sorted(range(len(load)), key=lambda e: (-load[e], e))
    if not world:
        return tuple(order[:slots])
    mean = sum(load) / world
    chosen: list = []
    while len(chosen) < slots and busiest_rank_load(load, world, chosen, placement, spread) > (1.0 + tolerance) * mean:
        chosen.append(order[len(chosen)])
    return tuple(chosen) + (-1,) * (slots - len(chosen))


def _allreduce_shadow_grads(ws: MoEWorkspace, grads):
    """Starts the sums; the returned handles are waited for once the rest of the backward pass has been enqueued."""
    if ws.heap.world > 1:
        import torch.distributed as dist
        return [dist.all_reduce(g, async_op=True, group=ws.reduce_group) for g in grads]
    return []


def _dispatch(ws: MoEWorkspace, x: torch.Tensor, idx: torch.Tensor, scale: Optional[torch.Tensor], dst, reuse: bool):
    C = require_native()
    h, cfg = ws.heap, ws.cfg
    if ws.slots_of is not None:
        j = (idx.clamp(-1, cfg.num_experts) + 1).long()
        idx = ws.slots_of[j]                                                    # expert id -> slot (see slot_table)
        if ws.spread is not None:
            idx = idx + ws.sh_stride[j] * ws.spread                             # a shadowed expert's copy on another rank
    C.moe_dispatch(x, idx, scale, ws.num_slots, ws.epr, ws.cap, h.rank, h.world, ws.local_count, ws.base, ws.pos,
                   ws.slot, ws.counts.peers(), ws.step_parity, dst.peers(), ws.info.peers(), reuse, h.status_addr)
    ws.launches += 1 if reuse else 2


def _wq(ws: MoEWorkspace, name: str, w: torch.Tensor):
    """(e4m3 buffer, scale buffer) of weight `name`, allocated on first use."""
    if name not in ws.wq:
        from . import fp8 as f8
        G, R, Cc = w.shape
        ws.wq[name] = (torch.empty(G, R, Cc, dtype=f8.FP8, device=w.device),
                       torch.empty(G, R // 128, Cc // 128, dtype=torch.float32, device=w.device))
    return ws.wq[name]


def moe_forward_dispatch(ws: MoEWorkspace, x: torch.Tensor, topk_idx: torch.Tensor) -> None:
    ws.step_parity = ws.parity
    ws.parity ^= 1
    _dispatch(ws, x, topk_idx, None, ws.xd, reuse=False)
    barrier(ws.heap, ws.name + ":d", signal=True, wait=False)
    ws.launches += 1


def moe_forward_experts(ws: MoEWorkspace, w13: torch.Tensor, w2: torch.Tensor) -> None:
    C = require_native()
    h = ws.heap
    barrier(h, ws.name + ":d", signal=False, wait=True)
    ws.copies_pending = False      # every rank's dispatch signal follows its writes into the copies (finish_shadow_grads)
    counts = ws.counts_now()
    C.moe_zero_tail(ws.xd.addr(), counts.data_ptr(), ws.epr, ws.cap, ws.cfg.hidden)
    st = h.status()
    if ws.cfg.fp8:
        from . import fp8 as f8
        C.fp8_quantize_blocks(w13, *_wq(ws, "w13", w13))
        C.fp8_quantize_blocks(w2, *_wq(ws, "w2", w2))
        C.fp8_quantize_rows(ws.xd.local, ws.q_in, ws.s_in, counts, ws.cap)
        f8.grouped_gemm_rows_fp8(ws.q_in, ws.s_in, *ws.wq["w13"], counts, ws.cap, epilogue=gemm.EPI_SWIGLU, out=ws.act,
                                 gu=ws.gu, zero_tail=True, status=st)
        C.fp8_quantize_rows(ws.act, ws.q_act, ws.s_act, counts, ws.cap)
        f8.grouped_gemm_rows_fp8(ws.q_act, ws.s_act, *ws.wq["w2"], counts, ws.cap, epilogue=gemm.EPI_SCATTER,
                                 row_info=ws.info.local, peers=ws.comb.peers(), ldc=ws.cfg.hidden, status=st, peer_rows=ws.comb.local.shape[0])
        ws.launches += 4
    else:
        gemm.grouped_gemm_rows(ws.xd.local, w13, counts, ws.cap, epilogue=gemm.EPI_SWIGLU, out=ws.act, gu=ws.gu,
                               zero_tail=True, status=st)
        gemm.grouped_gemm_rows(ws.act, w2, counts, ws.cap, epilogue=gemm.EPI_SCATTER, row_info=ws.info.local,
                               peers=ws.comb.peers(), ldc=ws.cfg.hidden, status=st, peer_rows=ws.comb.local.shape[0])
    barrier(h, ws.name + ":c", signal=True, wait=False)
    ws.launches += 5


def moe_forward_combine(ws: MoEWorkspace, topk_w: torch.Tensor) -> torch.Tensor:
    C = require_native()
    barrier(ws.heap, ws.name + ":c", signal=False, wait=True)
    out = torch.empty(ws.cfg.tokens, ws.cfg.hidden, dtype=torch.bfloat16, device=topk_w.device)
    C.moe_combine(ws.comb.local, topk_w, out, ws.cfg.topk)
    ws.launches += 2
    return out


def moe_backward_dispatch(ws: MoEWorkspace, dout: torch.Tensor, topk_idx: torch.Tensor, topk_w: torch.Tensor) -> torch.Tensor:
    """Phase 1 of backward: gate-weight gradient and dispatch of w_k * dOut to the slots chosen in forward."""
    C = require_native()
    cfg = ws.cfg
    dw = torch.empty(cfg.tokens, cfg.topk, dtype=torch.float32, device=dout.device)
    C.moe_combine_dw(dout, ws.comb.local, dw, cfg.topk)
    _dispatch(ws, dout, topk_idx, topk_w, ws.dyd, reuse=True)
    barrier(ws.heap, ws.name + ":bd", signal=True, wait=False)
    ws.launches += 2
    return dw


def moe_backward_experts(ws: MoEWorkspace, w13: torch.Tensor, w2: torch.Tensor, sgd_lr: float = 0.0,
                         need_dx: bool = True):
    """Phase 2: expert-side GEMMs.  Returns (dw13, dw2), both None when ``sgd_lr`` fuses the update."""
    C = require_native()
    h, cfg = ws.heap, ws.cfg
    barrier(h, ws.name + ":bd", signal=False, wait=True)
    counts = ws.counts_now()
    C.moe_zero_tail(ws.dyd.addr(), counts.data_ptr(), ws.epr, ws.cap, cfg.hidden)
    st = h.status()
    # dAct = dY @ W2 ; the epilogue turns it into dGate/dUp using the saved gate/up.  dX rows go home next (needs the
    # pre-update W13), then the weight gradients.
    overlap = bool(ws.overlap_reduce and ws.nshadow and ws.shadows_in_use and not cfg.fp8)
    beside = 0                                                       # CTAs a GEMM may use while the reduction's kernels run beside it
    if overlap and ws.dgu.device.type == "cuda":
        beside = max(2, (torch.cuda.get_device_properties(ws.dgu.device).multi_processor_count - ws.reduce_ctas - 4) // 2 * 2)
    if cfg.fp8:
        from . import fp8 as f8
        # the quantised weights of the forward pass are reused: a 128 x 128 scale block is its own transpose
        C.fp8_quantize_rows(ws.dyd.local, ws.q_in, ws.s_in, counts, ws.cap)
        f8.grouped_gemm_rows_fp8(ws.q_in, ws.s_in, *ws.wq["w2"], counts, ws.cap, b_mn_major=True, epilogue=gemm.EPI_DSWIGLU,
                                 gu=ws.gu, dgu=ws.dgu, zero_tail=True, status=st)
        if need_dx:
            C.fp8_quantize_rows(ws.dgu, ws.q_dgu, ws.s_dgu, counts, ws.cap)
            f8.grouped_gemm_rows_fp8(ws.q_dgu, ws.s_dgu, *ws.wq["w13"], counts, ws.cap, b_mn_major=True,
                                     epilogue=gemm.EPI_SCATTER, row_info=ws.info.local, peers=ws.dxs.peers(), ldc=cfg.hidden,
                                     status=st, peer_rows=ws.dxs.local.shape[0])
        ws.launches += 2
    else:
        gemm.grouped_gemm_rows(ws.dyd.local, w2, counts, ws.cap, b_mn_major=True, epilogue=gemm.EPI_DSWIGLU, gu=ws.gu,
                               dgu=ws.dgu, zero_tail=True, status=st)
        if overlap:
            # the copies' weight gradients first: their sum over the ranks starts now and runs beside what follows
            R, S, cut = ws.epr_real, ws.shadows_in_use, ws.epr_real * ws.cap
            end = cut + S * ws.cap
            early = (gemm.grouped_gemm_wgrad(ws.dgu[cut:end], ws.xd.local[cut:end], counts[R:R + S], ws.cap, S, status=st),
                     gemm.grouped_gemm_wgrad(ws.dyd.local[cut:end], ws.act[cut:end], counts[R:R + S], ws.cap, S, status=st))
            ws.launches += 2
            works = ws.reduce_shadow_grads(ws, early) or []
        if need_dx:
            gemm.grouped_gemm_rows(ws.dgu, w13, counts, ws.cap, b_mn_major=True, epilogue=gemm.EPI_SCATTER,
                                   row_info=ws.info.local, peers=ws.dxs.peers(), ldc=cfg.hidden, status=st,
                                   peer_rows=ws.dxs.local.shape[0], max_ctas=beside)
    shadow_grads = None
    if ws.nshadow:
        # Owned experts as below, on the leading slots.  The copies of the shadowed experts have seen this rank's rows
        # only: their gradients are stored, summed over the ranks after the signal and applied then, identically on
        # every rank, so the copies stay equal without ever being sent.
        R, S, cut = ws.epr_real, ws.shadows_in_use, ws.epr_real * ws.cap
        dyd, dgu, act, xd = ws.dyd.local, ws.dgu, ws.act, ws.xd.local
        if sgd_lr:
            gemm.grouped_gemm_wgrad(dyd[:cut], act[:cut], counts[:R], ws.cap, R, out=w2[:R], sgd_lr=sgd_lr, status=st, max_ctas=beside)
            gemm.grouped_gemm_wgrad(dgu[:cut], xd[:cut], counts[:R], ws.cap, R, out=w13[:R], sgd_lr=sgd_lr, status=st, max_ctas=beside)
            dw2 = dw13 = None
        else:
            dw2 = torch.empty_like(w2)
            dw13 = torch.empty_like(w13)
            gemm.grouped_gemm_wgrad(dyd[:cut], act[:cut], counts[:R], ws.cap, R, out=dw2[:R], status=st, max_ctas=beside)
            gemm.grouped_gemm_wgrad(dgu[:cut], xd[:cut], counts[:R], ws.cap, R, out=dw13[:R], status=st, max_ctas=beside)
            dw2[R:].zero_()                                          # copy slots: filled in once the sums are complete, empty
            dw13[R:].zero_()                                         # ones stay zero
        pk = ws.push
        if overlap:
            shadow_grads = early                                     # computed, and their reduction started, before dX
        elif S and pk is not None and ((sgd_lr and pk.w13 is not None and w13.data_ptr() == pk.w13.addr() and w2.data_ptr() == pk.w2.addr())
                                       or (not sgd_lr and pk.g13 is not None)):
            # the copies' gradient rows go from the GEMMs' epilogues to the ranks that sum them; moe_backward_finish
            # continues once every rank has signalled (shadow_update)
            end = cut + S * ws.cap
            gemm.grouped_gemm_wgrad_push(dgu[cut:end], xd[cut:end], counts[R:R + S], ws.cap, S, pk.p13.peers(), h.rank, pk.b13, status=st)
            gemm.grouped_gemm_wgrad_push(dyd[cut:end], act[cut:end], counts[R:R + S], ws.cap, S, pk.p2.peers(), h.rank, pk.b2, status=st)
            ws.launches += 2
            shadow_grads = S
        elif S:
            end = cut + S * ws.cap                                   # empty copy slots at the end take no part
            shadow_grads = (gemm.grouped_gemm_wgrad(dgu[cut:end], xd[cut:end], counts[R:R + S], ws.cap, S, status=st),
                            gemm.grouped_gemm_wgrad(dyd[cut:end], act[cut:end], counts[R:R + S], ws.cap, S, status=st))
            ws.launches += 2
    elif sgd_lr:
        gemm.grouped_gemm_wgrad(ws.dyd.local, ws.act, counts, ws.cap, ws.epr, out=w2, sgd_lr=sgd_lr, status=st)
        gemm.grouped_gemm_wgrad(ws.dgu, ws.xd.local, counts, ws.cap, ws.epr, out=w13, sgd_lr=sgd_lr, status=st)
        dw2 = dw13 = None
    else:
        dw2 = gemm.grouped_gemm_wgrad(ws.dyd.local, ws.act, counts, ws.cap, ws.epr, status=st)
        dw13 = gemm.grouped_gemm_wgrad(ws.dgu, ws.xd.local, counts, ws.cap, ws.epr, status=st)
    # every read of the buffers peers will overwrite next step is enqueued before this signal
    barrier(h, ws.name + ":bx", signal=True, wait=False)
    ws.launches += 6 + (1 if need_dx else 0)
    # finished in moe_backward_finish: the sum over ranks runs while the other ranks complete their GEMMs
    ws.pending_shadow = None if shadow_grads is None else (shadow_grads, w13, w2, dw13, dw2, sgd_lr)
    ws.started_shadow = works if (overlap and shadow_grads is not None) else None
    return dw13, dw2


def start_shadow_reduction(ws: MoEWorkspace):
    """Start summing the shadow experts' weight gradients over the ranks; returns what finish_shadow_grads needs."""
    if ws.pending_shadow is None:
        return None
    pending, ws.pending_shadow = ws.pending_shadow, None
    if ws.started_shadow is not None:                      # already running since the copies' gradients were computed
        works, ws.started_shadow = ws.started_shadow, None
    elif isinstance(pending[0], int):                      # pushed by the GEMMs: nothing to start
        works = []
    else:
        works = ws.reduce_shadow_grads(ws, pending[0]) or []
    return pending, works


def finish_shadow_grads(ws: MoEWorkspace, started) -> None:
    """With the sums complete: SGD on the copies (the same update on every rank, so they stay equal) or, without the fused
    update, the trailing slots of the gradients moe_backward_experts returned."""
    if started is None:
        return
    (grads, w13, w2, dw13, dw2, sgd_lr), works = started
    if isinstance(grads, int):
        # pushed: every rank's partial rows are in the staging (the callers wait for the ranks' signal first); sum the rows
        # this rank is responsible for, update them, and write them into every rank's copy
        S, R, pk, cfg, h = grads, ws.epr_real, ws.push, ws.cfg, ws.heap
        M13, N13, M2, N2 = 2 * cfg.ffn, cfg.hidden, cfg.hidden, cfg.ffn
        if sgd_lr:
            gemm.shadow_update(pk.p13.local, w13[R:], [a + R * M13 * N13 * 2 for a in pk.w13.peers()], S, h.rank, M13, N13, pk.b13,
                               M13 * N13, sgd_lr, pk.max_ctas)
            gemm.shadow_update(pk.p2.local, w2[R:], [a + R * M2 * N2 * 2 for a in pk.w2.peers()], S, h.rank, M2, N2, pk.b2,
                               M2 * N2, sgd_lr, pk.max_ctas)
            # This rank's copies are complete once EVERY rank has run the two kernels above.  The next forward pass learns
            # that from the ranks' dispatch signal, which each of them sends after this one; whatever else reads the copies
            # first (a change of shadows, a checkpoint) calls wait_for_copies.
            barrier(h, ws.name + ":bw", signal=True, wait=False)
            ws.copies_pending = True
            ws.launches += 1
        else:
            # the summed rows go into every rank's buffer; a rank's own buffer is complete once every rank has run this and
            # signalled
            gemm.shadow_update(pk.p13.local, None, pk.g13.peers(), S, h.rank, M13, N13, pk.b13, M13 * N13, 0.0, pk.max_ctas)
            gemm.shadow_update(pk.p2.local, None, pk.g2.peers(), S, h.rank, M2, N2, pk.b2, M2 * N2, 0.0, pk.max_ctas)
            barrier(h, ws.name + ":bg", signal=True, wait=False)
            ws.gathering_shadow = (S, dw13, dw2)              # moe_backward_complete waits for the ranks and fills dw13 / dw2
            ws.launches += 1
        ws.launches += 2
        return
    g13, g2 = grads
    for w in works:
        if hasattr(w, "wait"):
            w.wait()
    R, S = ws.epr_real, g13.shape[0]
    if sgd_lr:
        w13[R:R + S].add_(g13, alpha=-sgd_lr)
        w2[R:R + S].add_(g2, alpha=-sgd_lr)
    else:
        dw13[R:R + S].copy_(g13)
        dw2[R:R + S].copy_(g2)


def moe_backward_finish(ws: MoEWorkspace, need_dx: bool = True) -> Optional[torch.Tensor]:
    """Phase 3: wait for the returned input-gradient rows and sum them over k."""
    C = require_native()
    cfg = ws.cfg
    started = start_shadow_reduction(ws)          # runs beside the wait for the peers and the sum over k
    barrier(ws.heap, ws.name + ":bx", signal=False, wait=True)
    ws.launches += 1
    dx = None
    if need_dx:
        dx = torch.empty(cfg.tokens, cfg.hidden, dtype=torch.bfloat16, device=ws.dxs.local.device)
        C.moe_combine(ws.dxs.local, None, dx, cfg.topk)
        ws.launches += 1
    finish_shadow_grads(ws, started)
    return dx


def wait_for_copies(ws: MoEWorkspace) -> None:
    """After a step with the fused update of shadowed experts summed by this library: waits (on the current stream) until
    every rank has written the rows it updated into this rank's copies.  A no-op when nothing is outstanding."""
    if getattr(ws, "copies_pending", False):
        ws.copies_pending = False
        barrier(ws.heap, ws.name + ":bw", signal=False, wait=True)
        ws.launches += 1


def moe_backward_complete(ws: MoEWorkspace) -> None:
    """Phase 4, only where the copies' summed gradients are handed out (no fused update) and were summed by this library:
    once every rank has written the rows it summed into this rank's buffer, they are copied into the copy slots of the
    gradients moe_backward_experts returned."""
    pending = getattr(ws, "gathering_shadow", None)
    if pending is None:
        return
    ws.gathering_shadow = None
    S, dw13, dw2 = pending
    R, pk = ws.epr_real, ws.push
    barrier(ws.heap, ws.name + ":bg", signal=False, wait=True)
    dw13[R:R + S].copy_(pk.g13.local[:S])
    dw2[R:R + S].copy_(pk.g2.local[:S])
    ws.launches += 1


def moe_backward(ws: MoEWorkspace, dout: torch.Tensor, topk_idx: torch.Tensor, topk_w: torch.Tensor,
                 w13: torch.Tensor, w2: torch.Tensor, sgd_lr: float = 0.0, need_dx: bool = True):
    """Returns (dx, dtopk_w, dw13, dw2).  With ``sgd_lr`` the expert weights are updated in place by the wgrad
    kernels' epilogue and dw13/dw2 are None."""
    dw = moe_backward_dispatch(ws, dout.contiguous(), topk_idx, topk_w)
    dw13, dw2 = moe_backward_experts(ws, w13, w2, sgd_lr, need_dx)
    dx = moe_backward_finish(ws, need_dx)
    moe_backward_complete(ws)
    return dx, dw, dw13, dw2


class MoEFunction(torch.autograd.Function):
    """autograd node: (x, topk_w) are differentiable inputs, (w13, w2) differentiable parameters."""

    @staticmethod
    def forward(ctx, x, topk_w, topk_idx, w13, w2, ws: MoEWorkspace, sgd_lr: float):
        x = x.contiguous()
        topk_w = topk_w.contiguous().float()
        topk_idx = topk_idx.contiguous().int()
        moe_forward_dispatch(ws, x, topk_idx)
        moe_forward_experts(ws, w13, w2)
        out = moe_forward_combine(ws, topk_w)
        ctx.ws, ctx.sgd_lr = ws, sgd_lr
        ctx.save_for_backward(topk_w, topk_idx, w13, w2)
        ctx.need_dx = x.requires_grad
        return out

    @staticmethod
    def backward(ctx, dout):
        topk_w, topk_idx, w13, w2 = ctx.saved_tensors
        dx, dw, dw13, dw2 = moe_backward(ctx.ws, dout, topk_idx, topk_w, w13, w2, ctx.sgd_lr, need_dx=True)
        return dx, dw, None, dw13, dw2, None, None
