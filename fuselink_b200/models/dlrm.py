"""DLRM with table-wise sharded embeddings (the workload the reference runs through an external DLRM
checkout, .gitmodules:5-7).

Sparse side: 26 tables x rows x 128 fp32, sum pooling with a fixed pooling factor, tables spread over the
ranks.  The table owner pools the bags of the GLOBAL batch and its kernel stores each pooled vector
straight into the sample owner's ``[B_local, 26, 128]`` buffer (forward) / reads the gradient from there and
applies SGD to the rows (backward): csrc/kernels/embbag.cu.  Dense side (data parallel): bottom MLP
13-512-256-128, pairwise-dot interaction, top MLP 1024-1024-512-256-1, BCE-with-logits loss, SGD; dense
gradients are averaged with an NCCL all-reduce (not a named hot path).

On CPU tensors the same model runs as plain PyTorch (oracle and gloo tests).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .._ext import require_native
from ..ops import ref
from ..ops.comm import barrier
from ..parallel.symm import SymmetricHeap


@dataclass
class DLRMConfig:
    num_tables: int = 26
    rows: int = 1_000_000
    dim: int = 128
    pooling: int = 20
    dense_features: int = 13
    bottom: tuple = (512, 256, 128)
    top: tuple = (1024, 1024, 512, 256, 1)
    global_batch: int = 65536
    lr: float = 0.01
    zipf_alpha: float = 1.05


def table_split(num_tables: int, world: int) -> List[tuple]:
    """(first, count) of the tables each rank owns: 26 over 8 -> 4,4,3,3,3,3,3,3."""
    out, first = [], 0
    for r in range(world):
        n = num_tables // world + (1 if r < num_tables % world else 0)
        out.append((first, n))
        first += n
    return out


def zipf_indices(shape, rows: int, alpha: float, generator: torch.Generator, device) -> torch.Tensor:
    """Row ids with P(rank k) ~ k^-alpha over `rows` rows (inverse-CDF sampling of the continuous envelope)."""
    u = torch.rand(shape, generator=generator, device=device, dtype=torch.float64)
    if abs(alpha - 1.0) < 1e-9:
        k = torch.exp(u * torch.log(torch.tensor(float(rows) + 1.0, dtype=torch.float64, device=device)))
    else:
        a = 1.0 - alpha
        k = ((u * ((rows + 1.0) ** a - 1.0)) + 1.0) ** (1.0 / a)
    return (k.floor().long() - 1).clamp_(0, rows - 1)


def _mlp(sizes, last_act: bool) -> nn.Sequential:
    layers = []
    for i in range(len(sizes) - 1):
        layers.append(nn.Linear(sizes[i], sizes[i + 1]))
        if i < len(sizes) - 2 or last_act:
            layers.append(nn.ReLU())
    return nn.Sequential(*layers)


class DLRM(nn.Module):
    def __init__(self, cfg: DLRMConfig, heap: Optional[SymmetricHeap] = None, rank: int = 0, world: int = 1,
                 device="cuda", seed: int = 0, name: str = "dlrm"):
        super().__init__()
        self.cfg, self.rank, self.world, self.heap, self.name = cfg, rank, world, heap, name
        assert cfg.global_batch % world == 0
        self.b_local = cfg.global_batch // world
        self.t_first, self.t_local = table_split(cfg.num_tables, world)[rank]
        bound = cfg.rows ** -0.5
        g = torch.Generator(device="cpu").manual_seed(seed + 1)
        # tables: fp32 U(-1/sqrt(rows), 1/sqrt(rows)); each table's init depends only on its global index
        tabs = []
        for t in range(self.t_first, self.t_first + self.t_local):
            gt = torch.Generator(device=device if str(device) != "cpu" else "cpu").manual_seed(seed * 977 + t)
            tabs.append((torch.rand(cfg.rows, cfg.dim, generator=gt, device=device) * 2 - 1) * bound)
        # a buffer, not a Parameter: the backward kernel applies SGD to it in place; it is part of state_dict() for checkpoints
        self.register_buffer("tables", torch.stack(tabs) if tabs else torch.zeros(0, cfg.rows, cfg.dim, device=device))
        torch.manual_seed(seed)
        self.bottom = _mlp((cfg.dense_features,) + tuple(cfg.bottom), last_act=True).to(device)
        n_vec = cfg.num_tables + 1
        self.n_inter = n_vec * (n_vec - 1) // 2
        self.top = _mlp((self.n_inter + cfg.dim,) + tuple(cfg.top), last_act=False).to(device)
        iu = torch.triu_indices(n_vec, n_vec, offset=1)
        self.register_buffer("iu0", iu[0].to(device))
        self.register_buffer("iu1", iu[1].to(device))
        del g
        self.launches = 0
        if heap is not None:
            shape = [self.b_local, cfg.num_tables, cfg.dim]
            self.pooled = heap.alloc_tensor(shape, torch.float32)    # peers write pooled vectors here
            self.gpooled = heap.alloc_tensor(shape, torch.float32)   # peers read gradients from here

    # ---- sparse --------------------------------------------------------------------------------------------
    def sparse_forward_launch(self, indices: torch.Tensor):
        """indices: [t_local, B_global, pooling] int64 on this rank's device."""
        C = require_native()
        if self.t_local:
            C.embbag(False, self.tables, indices, self.t_first, self.cfg.num_tables, self.b_local, self.pooled.peers(), 0.0, 0,
                     self.heap.status_addr)
            self.launches += 1
        barrier(self.heap, self.name + ":f", signal=True, wait=False)
        self.launches += 1

    def sparse_forward_wait(self) -> torch.Tensor:
        barrier(self.heap, self.name + ":f", signal=False, wait=True)
        self.launches += 1
        return self.pooled.local

    def sparse_backward_launch(self, grad_pooled: torch.Tensor):
        self.gpooled.local.copy_(grad_pooled)
        barrier(self.heap, self.name + ":b", signal=True, wait=False)
        self.launches += 1

    def sparse_backward_apply(self, indices: torch.Tensor):
        C = require_native()
        barrier(self.heap, self.name + ":b", signal=False, wait=True)
        if self.t_local:
            C.embbag(True, self.tables, indices, self.t_first, self.cfg.num_tables, self.b_local, self.gpooled.peers(),
                     self.cfg.lr, 0, self.heap.status_addr)
            self.launches += 1
        # No trailing barrier is needed: a peer writes this rank's `pooled` for step s+1 only after its own wait on
        # ":b" of step s (which this rank signals after its dense backward), and this rank rewrites `gpooled` only
        # after its wait on ":f" of step s+1 (which peers signal after their step-s backward kernel).

    # ---- dense ---------------------------------------------------------------------------------------------
    def dense_forward(self, dense: torch.Tensor, pooled: torch.Tensor) -> torch.Tensor:
        x = self.bottom(dense)                                            # [B, dim]
        z = torch.cat([x.unsqueeze(1), pooled], dim=1)                    # [B, 27, dim]
        zz = torch.bmm(z, z.transpose(1, 2))                              # [B, 27, 27]
        inter = zz[:, self.iu0, self.iu1]
        return self.top(torch.cat([x, inter], dim=1)).squeeze(-1)

    def dense_parameters(self):
        return list(self.bottom.parameters()) + list(self.top.parameters())

    # ---- one training step (public API) --------------------------------------------------------------------
    def train_step(self, dense: torch.Tensor, indices: torch.Tensor, labels: torch.Tensor, opt: torch.optim.Optimizer):
        """Forward + backward + SGD on dense and sparse parameters.  Returns the (detached) loss."""
        fused = self.heap is not None          # a heap was given: the fused kernels (on host memory only in tests that model them)
        if fused:
            self.sparse_forward_launch(indices)
            pooled = self.sparse_forward_wait().detach().requires_grad_(True)
        else:
            pooled = self._pooled_reference(indices).requires_grad_(True)
        logits = self.dense_forward(dense, pooled)
        loss = F.binary_cross_entropy_with_logits(logits, labels)
        loss.backward()
        work = flat = grads = None
        if self.world > 1:
            # data-parallel part: one bucket for every dense gradient, reduced while the sparse backward runs
            import torch.distributed as dist
            from torch._utils import _flatten_dense_tensors, _unflatten_dense_tensors
            grads = [p.grad for p in self.dense_parameters()]
            flat = _flatten_dense_tensors(grads)
            work = dist.all_reduce(flat, async_op=True)
        # the loss is a mean over the local batch; the global objective is the mean over ranks
        gp = pooled.grad / self.world if self.world > 1 else pooled.grad
        if fused:
            self.sparse_backward_launch(gp)
            self.sparse_backward_apply(indices)
        else:
            self._sparse_backward_reference(indices, gp)
        if work is not None:
            work.wait()
            flat /= self.world
            for g, r in zip(grads, _unflatten_dense_tensors(flat, grads)):
                g.copy_(r)
        opt.step()
        opt.zero_grad(set_to_none=True)
        return loss.detach()

    # ---- CPU / gloo path -----------------------------------------------------------------------------------
    def _pooled_reference(self, indices):
        part = ref.embedding_bag_sum(self.tables, indices)                # [B_global, t_local, dim]
        if self.world == 1:
            return part
        import torch.distributed as dist
        full = torch.zeros(self.cfg.global_batch, self.cfg.num_tables, self.cfg.dim)
        full[:, self.t_first:self.t_first + self.t_local] = part
        dist.all_reduce(full)
        return full[self.rank * self.b_local:(self.rank + 1) * self.b_local].clone()

    def _sparse_backward_reference(self, indices, gp):
        if self.world == 1:
            g = gp
        else:
            import torch.distributed as dist
            full = torch.zeros(self.cfg.global_batch, self.cfg.num_tables, self.cfg.dim)
            full[self.rank * self.b_local:(self.rank + 1) * self.b_local] = gp
            dist.all_reduce(full)
            g = full
        ref.embedding_bag_sgd(self.tables, indices, g[:, self.t_first:self.t_first + self.t_local].contiguous(), self.cfg.lr)


def synthetic_batch(cfg: DLRMConfig, rank: int, world: int, device, seed: int):
    """(dense [B_local, 13], indices [t_local, B_global, pooling], labels [B_local]) for one step."""
    t_first, t_local = table_split(cfg.num_tables, world)[rank]
    b_local = cfg.global_batch // world
    g = torch.Generator(device=device).manual_seed(seed * 131 + rank)
    dense = torch.randn(b_local, cfg.dense_features, generator=g, device=device)
    labels = (torch.rand(b_local, generator=g, device=device) < 0.5).float()
    gi = torch.Generator(device=device).manual_seed(seed * 7919 + 13)
    # every rank derives the same global index tensor for a table from (seed, table), then keeps its tables
    idx = []
    for t in range(t_first, t_first + t_local):
        gt = torch.Generator(device=device).manual_seed(seed * 7919 + 13 + t)
        idx.append(zipf_indices((cfg.global_batch, cfg.pooling), cfg.rows, cfg.zipf_alpha, gt, device))
    del gi
    indices = torch.stack(idx) if idx else torch.zeros(0, cfg.global_batch, cfg.pooling, dtype=torch.long, device=device)
    return dense, indices, labels
