"""The stock formulation of the DLRM step used as the measured baseline: ``torch.nn.functional.embedding_bag``
per table, an NCCL ``all_to_all_single`` of the pooled embeddings (and of their gradients in backward), dense
autograd, and a sparse SGD update with ``index_add_``.  None of this library's kernels run here."""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .dlrm import DLRM, DLRMConfig


class BaselineDLRM(DLRM):
    def __init__(self, cfg: DLRMConfig, rank=0, world=1, device="cuda", seed=0):
        super().__init__(cfg, None, rank, world, device=device, seed=seed)
        from .dlrm import table_split
        self.split = table_split(cfg.num_tables, world)

    def train_step(self, dense, indices, labels, opt):
        import torch.distributed as dist
        cfg, W, bl = self.cfg, self.world, self.b_local
        Bg, L, D = cfg.global_batch, cfg.pooling, cfg.dim
        # forward: pool every local table over the global batch -> [B_global, t_local, D]
        pooled_parts = []
        for t in range(self.t_local):
            pooled_parts.append(F.embedding_bag(indices[t].reshape(-1), self.tables[t],
                                                torch.arange(0, Bg * L, L, device=dense.device), mode="sum"))
        mine = torch.stack(pooled_parts, 1) if pooled_parts else torch.zeros(Bg, 0, D, device=dense.device)
        if W > 1:
            send = mine.view(W, bl, self.t_local, D).contiguous()
            counts = [n for _, n in self.split]
            recv = torch.empty(bl * cfg.num_tables * D, device=dense.device)
            dist.all_to_all_single(recv, send.view(-1), [bl * n * D for n in counts], [bl * self.t_local * D] * W)
            chunks, o = [], 0
            for n in counts:
                chunks.append(recv[o:o + bl * n * D].view(bl, n, D))
                o += bl * n * D
            pooled = torch.cat(chunks, 1)
        else:
            pooled = mine
        pooled = pooled.detach().requires_grad_(True)
        logits = self.dense_forward(dense, pooled)
        loss = F.binary_cross_entropy_with_logits(logits, labels)
        loss.backward()
        if W > 1:
            for p in self.dense_parameters():
                dist.all_reduce(p.grad)
                p.grad /= W
            gp = pooled.grad / W
            counts = [n for _, n in self.split]
            send = torch.cat([gp[:, f:f + n].reshape(-1) for f, n in self.split])
            recv = torch.empty(Bg * self.t_local * D, device=dense.device)
            dist.all_to_all_single(recv, send, [bl * self.t_local * D] * W, [bl * n * D for n in counts])
            g = recv.view(W * bl, self.t_local, D)
        else:
            g = pooled.grad
        for t in range(self.t_local):
            gt = g[:, t].unsqueeze(1).expand(Bg, L, D).reshape(Bg * L, D)
            self.tables[t].index_add_(0, indices[t].reshape(-1), gt, alpha=-cfg.lr)
        opt.step()
        opt.zero_grad(set_to_none=True)
        return loss.detach()
