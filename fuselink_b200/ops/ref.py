"""Plain PyTorch fp32 restatements of every fused op; the oracles of the numerics tests and the CPU path
of the model layers (multi-process CPU tests run them over gloo)."""
from __future__ import annotations

import torch
import torch.nn.functional as F


def swiglu_ffn(x, w_gate, w_up, w_down):
    """x: [n, H]; w_gate/w_up: [F, H]; w_down: [H, F]; all computed in fp32."""
    x = x.float()
    return (F.silu(x @ w_gate.float().t()) * (x @ w_up.float().t())) @ w_down.float().t()


def moe_forward(x, topk_idx, topk_w, w_gate, w_up, w_down):
    """Dense oracle of a top-k MoE layer.  w_*: [E, ...].  Returns [T, H] fp32."""
    T, H = x.shape
    out = torch.zeros(T, H, dtype=torch.float32, device=x.device)
    for e in range(w_gate.shape[0]):
        tok, k = (topk_idx == e).nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        y = swiglu_ffn(x[tok], w_gate[e], w_up[e], w_down[e])
        out.index_add_(0, tok, y * topk_w[tok, k].float().unsqueeze(1))
    return out


def embedding_bag_sum(weights, indices):
    """weights: [T, rows, D]; indices: [T, B, L] -> [B, T, D] (sum pooling)."""
    T, B, L = indices.shape
    out = []
    for t in range(T):
        out.append(weights[t][indices[t].reshape(-1)].reshape(B, L, -1).sum(1))
    return torch.stack(out, dim=1)


def embedding_bag_sgd(weights, indices, grad, lr):
    """In-place SGD for sum-pooled bags: grad: [B, T, D]."""
    T, B, L = indices.shape
    for t in range(T):
        g = grad[:, t, :].unsqueeze(1).expand(B, L, -1).reshape(B * L, -1)
        weights[t].index_add_(0, indices[t].reshape(-1), g, alpha=-lr)
    return weights


def kv_gather_pages(pool, layout, block_table, num_blocks, layers, heads, block_size, head_dim):
    """Return the logical KV of each request as [layers, tokens, heads, head_dim] from a paged pool."""
    outs = []
    for b in range(block_table.shape[0]):
        pages = []
        for j in range(int(num_blocks[b])):
            blk = int(block_table[b, j])
            if layout == 0:   # [block][layer][head][slot][dim]
                p = pool.view(-1, layers, heads, block_size, head_dim)[blk].permute(0, 2, 1, 3)
            else:             # [layer][block][slot][head][dim]
                p = pool.view(layers, -1, block_size, heads, head_dim)[:, blk]
            pages.append(p)
        outs.append(torch.cat(pages, dim=1) if pages else pool.new_zeros(layers, 0, heads, head_dim))
    return outs
