"""Decoder-only transformers used by the disaggregated-serving path (prefill stage and decode stage): the
Llama family (RMSNorm, rotary positions, SwiGLU, no biases, grouped KV heads), the OPT family (pre-LayerNorm,
learned positions with an offset of 2, ReLU, biases, tied output embedding) and GPT-2 (as OPT with tanh-GELU and no
position offset) -- the three model families the reference's serving binary links (experiments/serving/
CMakeLists.txt:116-149: model_llama2, model_opt, model_gpt2).

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
    arch: str = "llama"          # "llama" | "opt" | "gpt2"
    max_pos: int = 4096          # rows of the learned position table (opt, gpt2)

    @property
    def pos_offset(self) -> int:
        return 2 if self.arch == "opt" else 0     # OPT's position table keeps two leading rows for padding ids


# name -> config: the model zoo of the reference's serving scripts plus the Llama-3-8B shape of the build target
MODEL_ZOO = {
    "llama3_8b": LlamaConfig(),
    "llama2_7b": LlamaConfig(layers=32, hidden=4096, heads=32, kv_heads=32, ffn=11008, vocab=32000, rope_theta=10000.0),
    "llama2_13b": LlamaConfig(layers=40, hidden=5120, heads=40, kv_heads=40, ffn=13824, vocab=32000, rope_theta=10000.0),
    "llama2_70b": LlamaConfig(layers=80, hidden=8192, heads=64, kv_heads=8, ffn=28672, vocab=32000, rope_theta=10000.0),
    "opt_125m": LlamaConfig(layers=12, hidden=768, heads=12, kv_heads=12, head_dim=64, ffn=3072, vocab=50272, arch="opt", max_pos=2048),
    "opt_1.3b": LlamaConfig(layers=24, hidden=2048, heads=32, kv_heads=32, head_dim=64, ffn=8192, vocab=50272, arch="opt", max_pos=2048),
    "opt_2.7b": LlamaConfig(layers=32, hidden=2560, heads=32, kv_heads=32, head_dim=80, ffn=10240, vocab=50272, arch="opt", max_pos=2048),
    "opt_6.7b": LlamaConfig(layers=32, hidden=4096, heads=32, kv_heads=32, ffn=16384, vocab=50272, arch="opt", max_pos=2048),
    "opt_13b": LlamaConfig(layers=40, hidden=5120, heads=40, kv_heads=40, ffn=20480, vocab=50272, arch="opt", max_pos=2048),
    "opt_30b": LlamaConfig(layers=48, hidden=7168, heads=56, kv_heads=56, ffn=28672, vocab=50272, arch="opt", max_pos=2048),
    "gpt2": LlamaConfig(layers=12, hidden=768, heads=12, kv_heads=12, head_dim=64, ffn=3072, vocab=50257, arch="gpt2", max_pos=1024),
    "gpt2_xl": LlamaConfig(layers=48, hidden=1600, heads=25, kv_heads=25, head_dim=64, ffn=6400, vocab=50257, arch="gpt2", max_pos=1024),
    "tiny": LlamaConfig(layers=2, hidden=256, heads=4, kv_heads=2, head_dim=64, ffn=512, vocab=1000),
    "tiny_opt": LlamaConfig(layers=2, hidden=256, heads=4, kv_heads=4, head_dim=64, ffn=512, vocab=1000, arch="opt", max_pos=512),
    "tiny_gpt2": LlamaConfig(layers=2, hidden=256, heads=4, kv_heads=4, head_dim=64, ffn=512, vocab=1000, arch="gpt2", max_pos=512),
}


def _rms(x, w, eps):
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * w


def _ln(x, w, b, eps):
    return F.layer_norm(x.float(), (x.shape[-1],), w.float(), b.float(), eps).to(x.dtype)


def _rope(x, pos, theta):
    """x: [..., n, heads, D]; pos: [..., n] absolute positions."""
    D = x.shape[-1]
    inv = 1.0 / (theta ** (torch.arange(0, D, 2, device=x.device, dtype=torch.float32) / D))
    ang = pos.float().unsqueeze(-1) * inv                      # [..., n, D/2]
    cos, sin = ang.cos().unsqueeze(-2), ang.sin().unsqueeze(-2)
    x1, x2 = x.float()[..., : D // 2], x.float()[..., D // 2:]
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], -1).to(x.dtype)


class LlamaShard(torch.nn.Module):
    """One tensor-parallel shard of the model.  ``tp_group`` is None for TP=1.  Column-parallel tensors (QKV, the first
    MLP matrix and their biases) are split over the shards, row-parallel ones (attention output, second MLP matrix) are
    reduced over the group and their biases added once after the reduction."""

    def __init__(self, cfg: LlamaConfig, tp_rank: int = 0, tp_size: int = 1, tp_group=None, device="cuda", seed: int = 0,
                 dtype=torch.bfloat16, max_positions: Optional[int] = None):
        super().__init__()
        assert cfg.heads % tp_size == 0 and cfg.kv_heads % tp_size == 0 and cfg.ffn % tp_size == 0
        assert cfg.arch in ("llama", "opt", "gpt2"), cfg.arch
        self.cfg, self.tp_rank, self.tp_size, self.tp_group = cfg, tp_rank, tp_size, tp_group
        self.h_local, self.kvh_local, self.f_local = cfg.heads // tp_size, cfg.kv_heads // tp_size, cfg.ffn // tp_size
        self.gated = cfg.arch == "llama"                                        # SwiGLU: gate and up in one matrix
        D, H = cfg.head_dim, cfg.hidden
        g = torch.Generator(device=device).manual_seed(seed * 31 + 7)           # replicated tensors: same on every shard
        gs = torch.Generator(device=device).manual_seed(seed * 31 + 100 + tp_rank)  # sharded tensors

        def w(shape, gen):
            return (torch.randn(*shape, generator=gen, device=device, dtype=torch.float32) * 0.02).to(dtype)

        def ones(n):
            return torch.ones(n, device=device, dtype=dtype)

        L = cfg.layers
        self.embed = w((cfg.vocab, H), g)
        self.lm_head = w((cfg.vocab, H), g) if cfg.arch == "llama" else self.embed    # OPT / GPT-2 tie the output embedding
        self.final_norm = ones(H)
        self.wqkv = [w(((self.h_local + 2 * self.kvh_local) * D, H), gs) for _ in range(L)]
        self.wo = [w((H, self.h_local * D), gs) for _ in range(L)]
        self.w13 = [w(((2 if self.gated else 1) * self.f_local, H), gs) for _ in range(L)]
        self.w2 = [w((H, self.f_local), gs) for _ in range(L)]
        self.n1 = [ones(H) for _ in range(L)]
        self.n2 = [ones(H) for _ in range(L)]
        none = [None] * L
        self.n1b, self.n2b, self.bqkv, self.bo, self.b13, self.b2 = none, none, none, none, none, none
        self.final_norm_b, self.pos_embed = None, None
        if cfg.arch != "llama":
            npos = max(cfg.max_pos, max_positions or 0) + cfg.pos_offset
            self.pos_embed = w((npos, H), g)
            self.final_norm_b = w((H,), g)
            self.n1b = [w((H,), g) for _ in range(L)]
            self.n2b = [w((H,), g) for _ in range(L)]
            self.bqkv = [w(((self.h_local + 2 * self.kvh_local) * D,), gs) for _ in range(L)]
            self.b13 = [w((self.f_local,), gs) for _ in range(L)]
            self.bo = [w((H,), g) for _ in range(L)]
            self.b2 = [w((H,), g) for _ in range(L)]

    # ------------------------------------------------------------------------------------------- building blocks
    def _allreduce(self, x):
        if self.tp_size > 1:
            import torch.distributed as dist
            dist.all_reduce(x, group=self.tp_group)
        return x

    def _norm(self, x, w, b):
        return _rms(x, w, self.cfg.eps) if b is None else _ln(x, w, b, self.cfg.eps)

    def _embed(self, tokens, pos):
        x = self.embed[tokens]
        if self.pos_embed is not None:
            x = x + self.pos_embed[pos + self.cfg.pos_offset]
        return x

    def _qkv(self, l, h, pos):
        """h: [..., n, H], pos: [..., n]  ->  q [..., n, h_local, D], k, v [..., n, kvh_local, D] (rotated for Llama)."""
        D = self.cfg.head_dim
        y = h @ self.wqkv[l].t()
        if self.bqkv[l] is not None:
            y = y + self.bqkv[l]
        qkv = y.view(*h.shape[:-1], self.h_local + 2 * self.kvh_local, D)
        q = qkv[..., : self.h_local, :]
        k = qkv[..., self.h_local: self.h_local + self.kvh_local, :]
        v = qkv[..., self.h_local + self.kvh_local:, :]
        if self.cfg.arch == "llama":
            q, k = _rope(q, pos, self.cfg.rope_theta), _rope(k, pos, self.cfg.rope_theta)
        return q, k, v

    def _attn_out(self, l, o):
        y = self._allreduce(o @ self.wo[l].t())
        return y if self.bo[l] is None else y + self.bo[l]

    def _mlp(self, l, x):
        h = x @ self.w13[l].t()
        if self.gated:
            a = F.silu(h[..., : self.f_local]) * h[..., self.f_local:]
        else:
            h = h + self.b13[l]
            a = F.relu(h) if self.cfg.arch == "opt" else F.gelu(h, approximate="tanh")
        y = self._allreduce(a @ self.w2[l].t())
        return y if self.b2[l] is None else y + self.b2[l]

    def _logits(self, x):
        return (self._norm(x, self.final_norm, self.final_norm_b) @ self.lm_head.t()).float()

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
        x = self._embed(tokens, pos)                                            # [B, S, H]
        for l in range(L):
            q, k, v = self._qkv(l, self._norm(x, self.n1[l], self.n1b[l]), pos)
            # page write: [B, S, h, D] -> [B*nblk, h, bs, D]
            kp[blocks, l] = k.reshape(B * nblk, bs, self.kvh_local, D).permute(0, 2, 1, 3)
            vp[blocks, l] = v.reshape(B * nblk, bs, self.kvh_local, D).permute(0, 2, 1, 3)
            if on_layer_done is not None:
                on_layer_done(l)                                                # KV of this layer may leave now
            o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True,
                                               enable_gqa=self.h_local != self.kvh_local)
            x = x + self._attn_out(l, o.transpose(1, 2).reshape(B, S, self.h_local * D))
            x = x + self._mlp(l, self._norm(x, self.n2[l], self.n2b[l]))
        xl = x[:, -1] if last_pos is None else x[torch.arange(B, device=x.device), last_pos]
        return self._logits(xl).argmax(-1)

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
        p1 = positions.unsqueeze(1)
        x = self._embed(tokens, positions)                                       # [B, H]
        for l in range(L):
            q, k, v = self._qkv(l, self._norm(x, self.n1[l], self.n1b[l]).unsqueeze(1), p1)   # [B, 1, heads, D]
            kp[l, cur_blk, cur_slot] = k[:, 0]
            vp[l, cur_blk, cur_slot] = v[:, 0]
            K = kp[l][bt].reshape(B, ctx, self.kvh_local, D)                     # gather this sequence's pages
            V = vp[l][bt].reshape(B, ctx, self.kvh_local, D)
            o = F.scaled_dot_product_attention(q.transpose(1, 2), K.transpose(1, 2), V.transpose(1, 2), attn_mask=mask,
                                               enable_gqa=self.h_local != self.kvh_local)
            x = x + self._attn_out(l, o.transpose(1, 2).reshape(B, self.h_local * D))
            x = x + self._mlp(l, self._norm(x, self.n2[l], self.n2b[l]))
        return self._logits(x).argmax(-1)

    # reference path for tests: full-sequence forward without paging, returns logits of the last position
    @torch.no_grad()
    def forward_dense(self, tokens: torch.Tensor, all_positions: bool = False) -> torch.Tensor:
        cfg = self.cfg
        B, S = tokens.shape
        D = cfg.head_dim
        pos = torch.arange(S, device=tokens.device).unsqueeze(0).expand(B, S)
        x = self._embed(tokens, pos)
        for l in range(cfg.layers):
            q, k, v = self._qkv(l, self._norm(x, self.n1[l], self.n1b[l]), pos)
            o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True,
                                               enable_gqa=self.h_local != self.kvh_local)
            x = x + self._attn_out(l, o.transpose(1, 2).reshape(B, S, self.h_local * D))
            x = x + self._mlp(l, self._norm(x, self.n2[l], self.n2b[l]))
        return self._logits(x if all_positions else x[:, -1])

    # ------------------------------------------------------------------------------------------- checkpoints
    def _hf_names(self, l: int):
        a = self.cfg.arch
        if a == "llama":
            pre = f"model.layers.{l}."
            return dict(q=pre + "self_attn.q_proj", k=pre + "self_attn.k_proj", v=pre + "self_attn.v_proj", o=pre + "self_attn.o_proj",
                        gate=pre + "mlp.gate_proj", up=pre + "mlp.up_proj", down=pre + "mlp.down_proj",
                        n1=pre + "input_layernorm", n2=pre + "post_attention_layernorm")
        if a == "opt":
            pre = f"model.decoder.layers.{l}."
            return dict(q=pre + "self_attn.q_proj", k=pre + "self_attn.k_proj", v=pre + "self_attn.v_proj", o=pre + "self_attn.out_proj",
                        up=pre + "fc1", down=pre + "fc2", n1=pre + "self_attn_layer_norm", n2=pre + "final_layer_norm")
        pre = f"transformer.h.{l}."
        return dict(qkv=pre + "attn.c_attn", o=pre + "attn.c_proj", up=pre + "mlp.c_fc", down=pre + "mlp.c_proj", n1=pre + "ln_1", n2=pre + "ln_2")

    _HF_TOP = {"llama": ("model.embed_tokens", None, "model.norm", "lm_head"),
               "opt": ("model.decoder.embed_tokens", "model.decoder.embed_positions", "model.decoder.final_layer_norm", "lm_head"),
               "gpt2": ("transformer.wte", "transformer.wpe", "transformer.ln_f", "lm_head")}

    @torch.no_grad()
    def load_hf_state_dict(self, sd: dict) -> None:
        """Fill this shard from a Hugging Face ``state_dict`` of the matching family (LlamaForCausalLM, OPTForCausalLM,
        GPT2LMHeadModel).  Column-parallel tensors are cut by head / by MLP column for this shard's ``tp_rank``, so every
        shard reads the same full checkpoint.  GPT-2 stores its projections transposed ([in, out])."""
        cfg, D = self.cfg, self.cfg.head_dim
        r, hl, kl, fl = self.tp_rank, self.h_local, self.kvh_local, self.f_local
        gpt2 = cfg.arch == "gpt2"

        def put(dst, src):
            assert dst.shape == src.shape, (tuple(dst.shape), tuple(src.shape))
            dst.copy_(src.to(device=dst.device, dtype=dst.dtype))

        def W(name):                                       # weight as [out, in]
            w = sd[name + ".weight"]
            return w.t() if gpt2 else w

        emb, pos, fin, head = self._HF_TOP[cfg.arch]
        put(self.embed, sd[emb + ".weight"])
        if cfg.arch == "llama":
            put(self.lm_head, sd.get(head + ".weight", sd[emb + ".weight"]))
        put(self.final_norm, sd[fin + ".weight"])
        if pos is not None:
            n = min(self.pos_embed.shape[0], sd[pos + ".weight"].shape[0])
            self.pos_embed[:n].copy_(sd[pos + ".weight"][:n].to(self.pos_embed.dtype))
            put(self.final_norm_b, sd[fin + ".bias"])
        for l in range(cfg.layers):
            nm = self._hf_names(l)
            if gpt2:
                wq, wk, wv = W(nm["qkv"]).split(cfg.hidden, 0)
                bq, bk, bv = sd[nm["qkv"] + ".bias"].split(cfg.hidden, 0)
            else:
                wq, wk, wv = W(nm["q"]), W(nm["k"]), W(nm["v"])
                if cfg.arch == "opt":
                    bq, bk, bv = (sd[nm[x] + ".bias"] for x in "qkv")
            put(self.wqkv[l], torch.cat([wq[r * hl * D:(r + 1) * hl * D], wk[r * kl * D:(r + 1) * kl * D], wv[r * kl * D:(r + 1) * kl * D]]))
            put(self.wo[l], W(nm["o"])[:, r * hl * D:(r + 1) * hl * D])
            put(self.w2[l], W(nm["down"])[:, r * fl:(r + 1) * fl])
            put(self.n1[l], sd[nm["n1"] + ".weight"])
            put(self.n2[l], sd[nm["n2"] + ".weight"])
            if self.gated:
                put(self.w13[l], torch.cat([W(nm["gate"])[r * fl:(r + 1) * fl], W(nm["up"])[r * fl:(r + 1) * fl]]))
            else:
                put(self.w13[l], W(nm["up"])[r * fl:(r + 1) * fl])
                put(self.b13[l], sd[nm["up"] + ".bias"][r * fl:(r + 1) * fl])
                put(self.bqkv[l], torch.cat([bq[r * hl * D:(r + 1) * hl * D], bk[r * kl * D:(r + 1) * kl * D], bv[r * kl * D:(r + 1) * kl * D]]))
                put(self.bo[l], sd[nm["o"] + ".bias"])
                put(self.b2[l], sd[nm["down"] + ".bias"])
                put(self.n1b[l], sd[nm["n1"] + ".bias"])
                put(self.n2b[l], sd[nm["n2"] + ".bias"])

    @torch.no_grad()
    def export_hf_state_dict(self) -> dict:
        """The inverse of :meth:`load_hf_state_dict` for an unsharded model (TP = 1)."""
        assert self.tp_size == 1, "gather the shards first"
        cfg, D = self.cfg, self.cfg.head_dim
        gpt2 = cfg.arch == "gpt2"
        sd = {}

        def outW(name, w):                                 # w is [out, in]
            sd[name + ".weight"] = (w.t() if gpt2 else w).contiguous().clone()

        emb, pos, fin, head = self._HF_TOP[cfg.arch]
        sd[emb + ".weight"] = self.embed.clone()
        sd[head + ".weight"] = self.lm_head.clone()
        sd[fin + ".weight"] = self.final_norm.clone()
        if pos is not None:
            sd[pos + ".weight"] = self.pos_embed.clone()
            sd[fin + ".bias"] = self.final_norm_b.clone()
        nq, nk = cfg.heads * D, cfg.kv_heads * D
        for l in range(cfg.layers):
            nm = self._hf_names(l)
            wq, wk, wv = self.wqkv[l].split([nq, nk, nk], 0)
            if gpt2:
                outW(nm["qkv"], self.wqkv[l])
                sd[nm["qkv"] + ".bias"] = self.bqkv[l].clone()
            else:
                outW(nm["q"], wq); outW(nm["k"], wk); outW(nm["v"], wv)
                if cfg.arch == "opt":
                    for x, b in zip("qkv", self.bqkv[l].split([nq, nk, nk], 0)):
                        sd[nm[x] + ".bias"] = b.clone()
            outW(nm["o"], self.wo[l])
            outW(nm["down"], self.w2[l])
            sd[nm["n1"] + ".weight"] = self.n1[l].clone()
            sd[nm["n2"] + ".weight"] = self.n2[l].clone()
            if self.gated:
                outW(nm["gate"], self.w13[l][: cfg.ffn]); outW(nm["up"], self.w13[l][cfg.ffn:])
            else:
                outW(nm["up"], self.w13[l])
                sd[nm["up"] + ".bias"] = self.b13[l].clone()
                sd[nm["o"] + ".bias"] = self.bo[l].clone()
                sd[nm["down"] + ".bias"] = self.b2[l].clone()
                sd[nm["n1"] + ".bias"] = self.n1b[l].clone()
                sd[nm["n2"] + ".bias"] = self.n2b[l].clone()
        return sd

    def state_dict_flat(self) -> dict:
        """Every tensor of this shard under a flat name (for ``torch.save``)."""
        out = {"embed": self.embed, "final_norm": self.final_norm}
        if self.lm_head is not self.embed:
            out["lm_head"] = self.lm_head
        for name in ("pos_embed", "final_norm_b"):
            if getattr(self, name) is not None:
                out[name] = getattr(self, name)
        for name in ("wqkv", "wo", "w13", "w2", "n1", "n2", "n1b", "n2b", "bqkv", "bo", "b13", "b2"):
            for l, t in enumerate(getattr(self, name)):
                if t is not None:
                    out[f"{name}.{l}"] = t
        return out

    @torch.no_grad()
    def load_state_dict_flat(self, sd: dict) -> None:
        mine = self.state_dict_flat()
        missing = set(mine) - set(sd)
        assert not missing, f"checkpoint lacks {sorted(missing)[:4]}"
        for k, t in mine.items():
            t.copy_(sd[k].to(device=t.device, dtype=t.dtype))


def load_checkpoint_file(path: str) -> dict:
    """A Hugging Face style ``state_dict`` from ``path``: a ``.pt`` / ``.bin`` file (``torch.load``), a ``.safetensors``
    file, or a directory holding any number of those shards."""
    import os
    if os.path.isdir(path):
        sd = {}
        for f in sorted(os.listdir(path)):
            if f.endswith((".pt", ".bin", ".safetensors")):
                sd.update(load_checkpoint_file(os.path.join(path, f)))
        if not sd:
            raise FileNotFoundError(f"no .pt / .bin / .safetensors file in {path}")
        return sd
    if path.endswith(".safetensors"):
        from safetensors.torch import load_file
        return load_file(path)
    sd = torch.load(path, map_location="cpu", weights_only=True)
    return sd.get("state_dict", sd) if isinstance(sd, dict) else sd


DecoderShard = LlamaShard      # the class serves every family of the zoo; the old name is kept for callers
