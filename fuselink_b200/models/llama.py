"""Llama-shaped decoder used by the disaggregated-serving path (prefill stage and decode stage).

The reference's serving experiment builds `st::model::Gpt<T>` from an external library with dummy weights
(experiments/serving/model.hh:165-177) and a table of model shapes (common_gpt_hyper_params.h:10-131).
Here the model is plain PyTorch (library attention / GEMMs: not a named hot path), tensor-parallel over a
process group, with random-init bf16 weights; what is hand-written is the KV hand-off between the stages
(csrc/kernels/kv_pack.cu), which this model feeds layer by layer through ``on_layer_done``.

Paged KV layouts (block = `block_size` tokens):
  prefill pool  [block][layer][head][slot][dim]   (FL_KV_BLHSD)
  decode pool   [layer][block][slot][head][dim]   (FL_KV_LBSHD)
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional

import torch
import torch.nn.functional as F

KV_BLHSD, KV_LBSHD = 0, 1


@dataclass
class LlamaConfig:
    layers: int = 32
    hidden: int = 4096
    heads: int = 32
    kv_heads: int = 8
    head_dim: int = 128
    ffn: int = 14336
    vocab: int = 128256
    rope_theta: float = 500000.0
    eps: float = 1e-5
    block_size: int = 16


# name -> config: the model zoo of the reference's serving scripts plus the Llama-3-8B shape of the build target
MODEL_ZOO = {
    "llama3_8b": LlamaConfig(),
    "llama2_7b": LlamaConfig(layers=32, hidden=4096, heads=32, kv_heads=32, ffn=11008, vocab=32000, rope_theta=10000.0),
    "llama2_13b": LlamaConfig(layers=40, hidden=5120, heads=40, kv_heads=40, ffn=13824, vocab=32000, rope_theta=10000.0),
    "llama2_70b": LlamaConfig(layers=80, hidden=8192, heads=64, kv_heads=8, ffn=28672, vocab=32000, rope_theta=10000.0),
    "opt_125m": LlamaConfig(layers=12, hidden=768, heads=12, kv_heads=12, head_dim=64, ffn=3072, vocab=50272),
    "opt_1.3b": LlamaConfig(layers=24, hidden=2048, heads=32, kv_heads=32, head_dim=64, ffn=8192, vocab=50272),
    "opt_2.7b": LlamaConfig(layers=32, hidden=2560, heads=32, kv_heads=32, head_dim=80, ffn=10240, vocab=50272),
    "opt_6.7b": LlamaConfig(layers=32, hidden=4096, heads=32, kv_heads=32, ffn=16384, vocab=50272),
    "opt_13b": LlamaConfig(layers=40, hidden=5120, heads=40, kv_heads=40, ffn=20480, vocab=50272),
    "opt_30b": LlamaConfig(layers=48, hidden=7168, heads=56, kv_heads=56, ffn=28672, vocab=50272),
    "tiny": LlamaConfig(layers=2, hidden=256, heads=4, kv_heads=2, head_dim=64, ffn=512, vocab=1000),
}


def _rms(x, w, eps):
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * w


def _rope(x, pos, theta):
    """x: [..., n, heads, D]; pos: [..., n] absolute positions."""
    D = x.shape[-1]
    inv = 1.0 / (theta ** (torch.arange(0, D, 2, device=x.device, dtype=torch.float32) / D))
    ang = pos.float().unsqueeze(-1) * inv                      # [..., n, D/2]
    cos, sin = ang.cos().unsqueeze(-2), ang.sin().unsqueeze(-2)
    x1, x2 = x.float()[..., : D // 2], x.float()[..., D // 2:]
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], -1).to(x.dtype)


class LlamaShard(torch.nn.Module):
    """One tensor-parallel shard of the model.  ``tp_group`` is None for TP=1."""

    def __init__(self, cfg: LlamaConfig, tp_rank: int = 0, tp_size: int = 1, tp_group=None, device="cuda", seed: int = 0,
                 dtype=torch.bfloat16):
        super().__init__()
        assert cfg.heads % tp_size == 0 and cfg.kv_heads % tp_size == 0 and cfg.ffn % tp_size == 0
        self.cfg, self.tp_rank, self.tp_size, self.tp_group = cfg, tp_rank, tp_size, tp_group
        self.h_local, self.kvh_local, self.f_local = cfg.heads // tp_size, cfg.kv_heads // tp_size, cfg.ffn // tp_size
        D, H = cfg.head_dim, cfg.hidden
        g = torch.Generator(device=device).manual_seed(seed * 31 + 7)           # replicated tensors: same on every shard
        gs = torch.Generator(device=device).manual_seed(seed * 31 + 100 + tp_rank)  # sharded tensors

        def w(shape, gen):
            return (torch.randn(*shape, generator=gen, device=device, dtype=torch.float32) * 0.02).to(dtype)

        self.embed = w((cfg.vocab, H), g)
        self.lm_head = w((cfg.vocab, H), g)
        self.final_norm = torch.ones(H, device=device, dtype=dtype)
        self.wqkv = [w(((self.h_local + 2 * self.kvh_local) * D, H), gs) for _ in range(cfg.layers)]
        self.wo = [w((H, self.h_local * D), gs) for _ in range(cfg.layers)]
        self.w13 = [w((2 * self.f_local, H), gs) for _ in range(cfg.layers)]
        self.w2 = [w((H, self.f_local), gs) for _ in range(cfg.layers)]
        self.n1 = [torch.ones(H, device=device, dtype=dtype) for _ in range(cfg.layers)]
        self.n2 = [torch.ones(H, device=device, dtype=dtype) for _ in range(cfg.layers)]

    def _allreduce(self, x):
        if self.tp_size > 1:
            import torch.distributed as dist
            dist.all_reduce(x, group=self.tp_group)
        return x

    def _mlp(self, l, x):
        h = x @ self.w13[l].t()
        a = F.silu(h[..., : self.f_local]) * h[..., self.f_local:]
        return self._allreduce(a @ self.w2[l].t())

    # ------------------------------------------------------------------------------------------- prefill
    @torch.no_grad()
    def prefill(self, tokens: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, block_table: torch.Tensor,
                on_layer_done: Optional[Callable[[int], None]] = None, last_pos: Optional[torch.Tensor] = None) -> torch.Tensor:
        """tokens: [B, S] (S a multiple of block_size); pools: flat bf16 in the BLHSD layout; block_table: [B, >=S/bs]
        int32.  Fills the pools, returns the greedy first token of every sequence [B] (int64)."""
        cfg = self.cfg
        B, S = tokens.shape
        bs, D, L = cfg.block_size, cfg.head_dim, cfg.layers
        assert S % bs == 0
        nblk = S // bs
        kp = k_pool.view(-1, L, self.kvh_local, bs, D)
        vp = v_pool.view(-1, L, self.kvh_local, bs, D)
        blocks = block_table[:, :nblk].long().reshape(-1)                       # [B*nblk]
        pos = torch.arange(S, device=tokens.device).unsqueeze(0).expand(B, S)
        x = self.embed[tokens]                                                  # [B, S, H]
        for l in range(L):
            h = _rms(x, self.n1[l], cfg.eps)
            qkv = (h @ self.wqkv[l].t()).view(B, S, self.h_local + 2 * self.kvh_local, D)
            q = _rope(qkv[:, :, : self.h_local], pos, cfg.rope_theta)
            k = _rope(qkv[:, :, self.h_local: self.h_local + self.kvh_local], pos, cfg.rope_theta)
            v = qkv[:, :, self.h_local + self.kvh_local:]
            # page write: [B, S, h, D] -> [B*nblk, h, bs, D]
            kp[blocks, l] = k.reshape(B * nblk, bs, self.kvh_local, D).permute(0, 2, 1, 3)
            vp[blocks, l] = v.reshape(B * nblk, bs, self.kvh_local, D).permute(0, 2, 1, 3)
            if on_layer_done is not None:
                on_layer_done(l)                                                # KV of this layer may leave now
            o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True,
                                               enable_gqa=self.h_local != self.kvh_local)
            x = x + self._allreduce(o.transpose(1, 2).reshape(B, S, self.h_local * D) @ self.wo[l].t())
            x = x + self._mlp(l, _rms(x, self.n2[l], cfg.eps))
        xl = x[:, -1] if last_pos is None else x[torch.arange(B, device=x.device), last_pos]
        last = _rms(xl, self.final_norm, cfg.eps)
        return (last @ self.lm_head.t()).float().argmax(-1)

    # ------------------------------------------------------------------------------------------- decode
    @torch.no_grad()
    def decode_step(self, tokens: torch.Tensor, positions: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                    block_table: torch.Tensor, num_pool_blocks: int) -> torch.Tensor:
        """One greedy step for B sequences.  tokens, positions: [B]; pools: flat bf16 in the LBSHD layout;
        block_table: [B, max_blocks] int32 covering position + 1 tokens.  Returns next tokens [B]."""
        cfg = self.cfg
        B = tokens.shape[0]
        bs, D, L = cfg.block_size, cfg.head_dim, cfg.layers
        kp = k_pool.view(L, num_pool_blocks, bs, self.kvh_local, D)
        vp = v_pool.view(L, num_pool_blocks, bs, self.kvh_local, D)
        bt = block_table.long()
        maxblk = bt.shape[1]
        ar = torch.arange(B, device=tokens.device)
        cur_blk = bt[ar, positions // bs]
        cur_slot = positions % bs
        ctx = maxblk * bs
        mask = (torch.arange(ctx, device=tokens.device).unsqueeze(0) <= positions.unsqueeze(1)).view(B, 1, 1, ctx)
        x = self.embed[tokens]                                                   # [B, H]
        for l in range(L):
            h = _rms(x, self.n1[l], cfg.eps)
            qkv = (h @ self.wqkv[l].t()).view(B, 1, self.h_local + 2 * self.kvh_local, D)
            p1 = positions.unsqueeze(1)
            q = _rope(qkv[:, :, : self.h_local], p1, cfg.rope_theta)
            k = _rope(qkv[:, :, self.h_local: self.h_local + self.kvh_local], p1, cfg.rope_theta)
            v = qkv[:, :, self.h_local + self.kvh_local:]
            kp[l, cur_blk, cur_slot] = k[:, 0]
            vp[l, cur_blk, cur_slot] = v[:, 0]
            K = kp[l][bt].reshape(B, ctx, self.kvh_local, D)                     # gather this sequence's pages
            V = vp[l][bt].reshape(B, ctx, self.kvh_local, D)
            o = F.scaled_dot_product_attention(q.transpose(1, 2), K.transpose(1, 2), V.transpose(1, 2), attn_mask=mask,
                                               enable_gqa=self.h_local != self.kvh_local)
            x = x + self._allreduce(o.transpose(1, 2).reshape(B, self.h_local * D) @ self.wo[l].t())
            x = x + self._mlp(l, _rms(x, self.n2[l], cfg.eps))
        return (_rms(x, self.final_norm, cfg.eps) @ self.lm_head.t()).float().argmax(-1)

    # reference path for tests: full-sequence forward without paging, returns logits of the last position
    @torch.no_grad()
    def forward_dense(self, tokens: torch.Tensor) -> torch.Tensor:
        cfg = self.cfg
        B, S = tokens.shape
        D = cfg.head_dim
        pos = torch.arange(S, device=tokens.device).unsqueeze(0).expand(B, S)
        x = self.embed[tokens]
        for l in range(cfg.layers):
            h = _rms(x, self.n1[l], cfg.eps)
            qkv = (h @ self.wqkv[l].t()).view(B, S, self.h_local + 2 * self.kvh_local, D)
            q = _rope(qkv[:, :, : self.h_local], pos, cfg.rope_theta)
            k = _rope(qkv[:, :, self.h_local: self.h_local + self.kvh_local], pos, cfg.rope_theta)
            v = qkv[:, :, self.h_local + self.kvh_local:]
            o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True,
                                               enable_gqa=self.h_local != self.kvh_local)
            x = x + self._allreduce(o.transpose(1, 2).reshape(B, S, self.h_local * D) @ self.wo[l].t())
            x = x + self._mlp(l, _rms(x, self.n2[l], cfg.eps))
        return (_rms(x[:, -1], self.final_norm, cfg.eps) @ self.lm_head.t()).float()
