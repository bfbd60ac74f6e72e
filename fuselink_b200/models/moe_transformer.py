"""A decoder-only transformer whose feed-forward blocks are expert-parallel MoE layers (Mixtral-shaped): the kind of
model the reference's expert-parallel experiment trains through Megatron-DeepSpeed (.gitmodules:11-13).

Parallelism, as in that setup: the experts of every layer are spread over the ranks (EP = world) and exchanged through
:class:`~fuselink_b200.models.moe.MoELayer` (fused dispatch / grouped GEMM / combine on CUDA); everything else --
embeddings, attention, norms, routers, output head -- is replicated and its gradients are averaged over the ranks (DP)
in one bucket.  Every rank feeds its own micro-batch.

The attention and the dense GEMMs are library calls (``scaled_dot_product_attention``, ``matmul``); the hand-written
kernels are the ones inside the MoE layer.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops.moe import MoEConfig
from ..parallel.symm import SymmetricHeap
from .llama import _rms, _rope
from .moe import MoELayer


@dataclass
class MoEModelConfig:
    layers: int = 32
    hidden: int = 4096
    heads: int = 32
    kv_heads: int = 8
    head_dim: int = 128
    ffn: int = 14336
    num_experts: int = 8
    topk: int = 2
    vocab: int = 32000
    rope_theta: float = 1e6
    eps: float = 1e-5
    aux_loss_coef: float = 0.01
    capacity_factor: float = 0.0          # > 0 with drop_tokens: choices over an expert's capacity contribute nothing
    drop_tokens: bool = False
    placement: Optional[str] = None       # "balanced": experts' homes evened out by the router's bias (MoELayer)
    shadow_experts: int = 0               # copies of the n experts the router favours most on every rank (CUDA path)


MOE_ZOO = {
    "mixtral_8x7b": MoEModelConfig(),
    "tiny_moe": MoEModelConfig(layers=2, hidden=128, heads=4, kv_heads=2, head_dim=32, ffn=256, num_experts=4, topk=2, vocab=512),
}


class _Block(nn.Module):
    def __init__(self, cfg: MoEModelConfig, moe: MoELayer, device, gen: torch.Generator, dtype):
        super().__init__()
        H, D = cfg.hidden, cfg.head_dim

        def w(*shape):
            return nn.Parameter((torch.randn(*shape, generator=gen) * 0.02).to(dtype).to(device))

        self.cfg = cfg
        self.wqkv = w((cfg.heads + 2 * cfg.kv_heads) * D, H)
        self.wo = w(H, cfg.heads * D)
        self.n1 = nn.Parameter(torch.ones(H, dtype=dtype, device=device))
        self.n2 = nn.Parameter(torch.ones(H, dtype=dtype, device=device))
        self.moe = moe

    def forward(self, x: torch.Tensor, pos: torch.Tensor) -> torch.Tensor:
        cfg = self.cfg
        B, S, H = x.shape
        D = cfg.head_dim
        h = _rms(x, self.n1, cfg.eps)
        qkv = (h @ self.wqkv.t()).view(B, S, cfg.heads + 2 * cfg.kv_heads, D)
        q = _rope(qkv[:, :, : cfg.heads], pos, cfg.rope_theta)
        k = _rope(qkv[:, :, cfg.heads: cfg.heads + cfg.kv_heads], pos, cfg.rope_theta)
        v = qkv[:, :, cfg.heads + cfg.kv_heads:]
        o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True,
                                           enable_gqa=cfg.heads != cfg.kv_heads)
        x = x + o.transpose(1, 2).reshape(B, S, cfg.heads * D) @ self.wo.t()
        y = self.moe(_rms(x, self.n2, cfg.eps).reshape(B * S, H))          # tokens of this rank go to the experts' owners
        return x + y.view(B, S, H)


class MoETransformer(nn.Module):
    """``tokens_per_rank`` = batch x sequence of one step on one rank (the MoE workspaces are sized for it)."""

    def __init__(self, cfg: MoEModelConfig, tokens_per_rank: int, heap: Optional[SymmetricHeap] = None, rank: int = 0,
                 world: int = 1, device="cuda", seed: int = 0, dtype=torch.bfloat16, fused_sgd_lr: float = 0.0):
        super().__init__()
        self.cfg, self.rank, self.world = cfg, rank, world
        gen = torch.Generator().manual_seed(seed * 7919 + 13)              # replicated parameters: same on every rank
        self.embed = nn.Parameter((torch.randn(cfg.vocab, cfg.hidden, generator=gen) * 0.02).to(dtype).to(device))
        self.lm_head = nn.Parameter((torch.randn(cfg.vocab, cfg.hidden, generator=gen) * 0.02).to(dtype).to(device))
        self.final_norm = nn.Parameter(torch.ones(cfg.hidden, dtype=dtype, device=device))
        mcfg = MoEConfig(hidden=cfg.hidden, ffn=cfg.ffn, num_experts=cfg.num_experts, topk=cfg.topk, tokens=tokens_per_rank)
        blocks = []
        for l in range(cfg.layers):
            moe = MoELayer(mcfg, heap, rank, world, device=device, zipf_s=None, seed=seed * 100 + l, fused_sgd_lr=fused_sgd_lr,
                           name=f"moe{l}", capacity_factor=cfg.capacity_factor, drop_tokens=cfg.drop_tokens,
                           shadow_experts=cfg.shadow_experts if world > 1 else 0, placement=cfg.placement)
            blocks.append(_Block(cfg, moe, device, gen, dtype))
        self.blocks = nn.ModuleList(blocks)

    # ---- parameters by parallelism ------------------------------------------------------------------------
    def expert_parameters(self) -> List[nn.Parameter]:
        return [p for b in self.blocks for p in (b.moe.w13, b.moe.w2)]

    def dense_parameters(self) -> List[nn.Parameter]:
        experts = {id(p) for p in self.expert_parameters()}
        return [p for p in self.parameters() if id(p) not in experts]

    # ---- forward / loss -------------------------------------------------------------------------------------
    def forward(self, tokens: torch.Tensor) -> torch.Tensor:
        B, S = tokens.shape
        pos = torch.arange(S, device=tokens.device).unsqueeze(0).expand(B, S)
        x = self.embed[tokens]
        for b in self.blocks:
            x = b(x, pos)
        return (_rms(x, self.final_norm, self.cfg.eps) @ self.lm_head.t()).float()

    def loss(self, tokens: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
        """Next-token cross entropy plus the load-balancing term of every MoE layer."""
        logits = self(tokens)
        ce = F.cross_entropy(logits.view(-1, logits.shape[-1]), labels.reshape(-1))
        aux = sum(b.moe.l_aux for b in self.blocks) / len(self.blocks)
        return ce + self.cfg.aux_loss_coef * aux

    def allreduce_dense_grads(self) -> None:
        """Data-parallel average of the replicated parameters' gradients, one bucket (expert gradients stay local)."""
        if self.world == 1:
            return
        import torch.distributed as dist
        from torch._utils import _flatten_dense_tensors, _unflatten_dense_tensors
        grads = [p.grad for p in self.dense_parameters() if p.grad is not None]
        flat = _flatten_dense_tensors(grads)
        dist.all_reduce(flat)
        flat /= self.world
        for g, r in zip(grads, _unflatten_dense_tensors(flat, grads)):
            g.copy_(r)

    def train_step(self, tokens: torch.Tensor, labels: torch.Tensor, opt: torch.optim.Optimizer) -> torch.Tensor:
        loss = self.loss(tokens, labels)
        loss.backward()
        self.allreduce_dense_grads()
        opt.step()
        opt.zero_grad(set_to_none=True)
        return loss.detach()
