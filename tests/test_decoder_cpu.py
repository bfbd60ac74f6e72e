"""The decoder families of the serving path (Llama, OPT, GPT-2) on the CPU in fp32:
  * logits equal those of the Hugging Face implementation of the same family carrying the same weights (export and
    load direction), which pins the architecture details: norm type, position scheme, activation, biases, tied head;
  * paged prefill + decode steps reproduce the dense forward (greedy tokens), per family;
  * two tensor-parallel shards cut from one checkpoint reproduce the unsharded model (gloo ranks)."""
import os
import socket
import tempfile

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from fuselink_b200.models.llama import MODEL_ZOO, LlamaConfig, LlamaShard

FAMILIES = ["tiny", "tiny_opt", "tiny_gpt2"]


def _hf_model(cfg: LlamaConfig):
    tr = pytest.importorskip("transformers")
    if cfg.arch == "llama":
        c = tr.LlamaConfig(vocab_size=cfg.vocab, hidden_size=cfg.hidden, intermediate_size=cfg.ffn, num_hidden_layers=cfg.layers,
                           num_attention_heads=cfg.heads, num_key_value_heads=cfg.kv_heads, head_dim=cfg.head_dim,
                           rms_norm_eps=cfg.eps, rope_theta=cfg.rope_theta, max_position_embeddings=2048,
                           attention_bias=False, mlp_bias=False, tie_word_embeddings=False, hidden_act="silu")
        return tr.LlamaForCausalLM(c)
    if cfg.arch == "opt":
        c = tr.OPTConfig(vocab_size=cfg.vocab, hidden_size=cfg.hidden, ffn_dim=cfg.ffn, num_hidden_layers=cfg.layers,
                         num_attention_heads=cfg.heads, max_position_embeddings=cfg.max_pos, word_embed_proj_dim=cfg.hidden,
                         do_layer_norm_before=True, activation_function="relu", dropout=0.0, attention_dropout=0.0,
                         layerdrop=0.0, enable_bias=True, layer_norm_elementwise_affine=True)
        return tr.OPTForCausalLM(c)
    c = tr.GPT2Config(vocab_size=cfg.vocab, n_embd=cfg.hidden, n_inner=cfg.ffn, n_layer=cfg.layers, n_head=cfg.heads,
                      n_positions=cfg.max_pos, activation_function="gelu_new", layer_norm_epsilon=cfg.eps,
                      resid_pdrop=0.0, embd_pdrop=0.0, attn_pdrop=0.0)
    return tr.GPT2LMHeadModel(c)


def _randomise(net: LlamaShard, seed: int):
    """Norm gains / biases away from their 1 / 0 initial values so that a swapped or dropped tensor shows."""
    g = torch.Generator().manual_seed(seed)
    for t in net.state_dict_flat().values():
        if t.dim() == 1:
            t.add_(torch.randn(t.shape, generator=g) * 0.1)


@pytest.mark.parametrize("name", FAMILIES)
def test_logits_match_hugging_face_with_exported_weights(name):
    cfg = MODEL_ZOO[name]
    net = LlamaShard(cfg, device="cpu", dtype=torch.float32, seed=3)
    _randomise(net, 1)
    hf = _hf_model(cfg).eval()
    sd = net.export_hf_state_dict()
    res = hf.load_state_dict(sd, strict=False)
    assert not res.unexpected_keys, res.unexpected_keys
    # what may be absent from the export: buffers (rotary tables, causal masks) and a tied head alias
    assert all(("rotary" in k or "inv_freq" in k or k.endswith(".attn.bias") or k.endswith("masked_bias")) for k in res.missing_keys), res.missing_keys
    tokens = torch.randint(0, cfg.vocab, (2, 48), generator=torch.Generator().manual_seed(5))
    with torch.no_grad():
        want = hf(input_ids=tokens).logits
    got = net.forward_dense(tokens, all_positions=True)
    assert got.shape == want.shape
    assert (got - want).abs().max() < 2e-4 * max(1.0, want.abs().max().item()), (got - want).abs().max()


@pytest.mark.parametrize("name", FAMILIES)
def test_loading_a_hugging_face_checkpoint(name):
    cfg = MODEL_ZOO[name]
    torch.manual_seed(11)
    hf = _hf_model(cfg).eval()
    net = LlamaShard(cfg, device="cpu", dtype=torch.float32, seed=0)
    net.load_hf_state_dict(hf.state_dict())
    tokens = torch.randint(0, cfg.vocab, (1, 33), generator=torch.Generator().manual_seed(6))
    with torch.no_grad():
        want = hf(input_ids=tokens).logits[:, -1]
    got = net.forward_dense(tokens)
    assert (got - want).abs().max() < 2e-4 * max(1.0, want.abs().max().item())


@pytest.mark.parametrize("name", FAMILIES)
def test_paged_prefill_and_decode_follow_the_dense_model(name):
    cfg = MODEL_ZOO[name]
    net = LlamaShard(cfg, device="cpu", dtype=torch.float32, seed=2)
    _randomise(net, 2)
    B, S, steps, bs = 2, 32, 5, cfg.block_size
    nblk_max = (S + steps + bs - 1) // bs
    nblocks = B * nblk_max + 3
    perm = torch.randperm(nblocks, generator=torch.Generator().manual_seed(3))[: B * nblk_max].view(B, nblk_max).int()
    elems = nblocks * cfg.layers * cfg.kv_heads * bs * cfg.head_dim
    kp, vp = torch.zeros(elems), torch.zeros(elems)
    tokens = torch.randint(0, cfg.vocab, (B, S), generator=torch.Generator().manual_seed(4))
    first = net.prefill(tokens, kp, vp, perm)
    assert torch.equal(first, net.forward_dense(tokens).argmax(-1))
    # hand the pages to the decode layout [layer][block][slot][head][dim]
    L, H, D = cfg.layers, cfg.kv_heads, cfg.head_dim
    kd = kp.view(nblocks, L, H, bs, D).permute(1, 0, 3, 2, 4).contiguous().view(-1)
    vd = vp.view(nblocks, L, H, bs, D).permute(1, 0, 3, 2, 4).contiguous().view(-1)
    seq = torch.cat([tokens, first.unsqueeze(1)], 1)
    for t in range(steps):
        pos = torch.full((B,), S + t, dtype=torch.long)
        nxt = net.decode_step(seq[:, -1], pos, kd, vd, perm, nblocks)
        want = net.forward_dense(seq).argmax(-1)
        assert torch.equal(nxt, want), (name, t)
        seq = torch.cat([seq, nxt.unsqueeze(1)], 1)


@pytest.mark.parametrize("name", FAMILIES)
def test_paged_path_runs_in_bf16(name):
    """The serving dtype: every family goes through paged prefill and decode in bf16 without a dtype mismatch (norms in
    fp32, everything else in bf16) and still mostly agrees with its own dense forward."""
    cfg = MODEL_ZOO[name]
    net = LlamaShard(cfg, device="cpu", dtype=torch.bfloat16, seed=2)
    B, S, steps, bs = 2, 32, 3, cfg.block_size
    nblk_max = (S + steps + bs - 1) // bs
    nblocks = B * nblk_max + 3
    perm = torch.randperm(nblocks, generator=torch.Generator().manual_seed(3))[: B * nblk_max].view(B, nblk_max).int()
    elems = nblocks * cfg.layers * cfg.kv_heads * bs * cfg.head_dim
    kp, vp = torch.zeros(elems, dtype=torch.bfloat16), torch.zeros(elems, dtype=torch.bfloat16)
    tokens = torch.randint(0, cfg.vocab, (B, S), generator=torch.Generator().manual_seed(4))
    first = net.prefill(tokens, kp, vp, perm)
    L, H, D = cfg.layers, cfg.kv_heads, cfg.head_dim
    kd = kp.view(nblocks, L, H, bs, D).permute(1, 0, 3, 2, 4).contiguous().view(-1)
    vd = vp.view(nblocks, L, H, bs, D).permute(1, 0, 3, 2, 4).contiguous().view(-1)
    seq = torch.cat([tokens, first.unsqueeze(1)], 1)
    agree = 0
    for t in range(steps):
        nxt = net.decode_step(seq[:, -1], torch.full((B,), S + t, dtype=torch.long), kd, vd, perm, nblocks)
        agree += int((nxt == net.forward_dense(seq).argmax(-1)).sum())
        seq = torch.cat([seq, nxt.unsqueeze(1)], 1)
    assert agree >= steps * B // 2


def test_flat_checkpoint_round_trip():
    cfg = MODEL_ZOO["tiny_opt"]
    a = LlamaShard(cfg, device="cpu", dtype=torch.float32, seed=1)
    b = LlamaShard(cfg, device="cpu", dtype=torch.float32, seed=9)
    with tempfile.TemporaryDirectory() as d:
        torch.save(a.state_dict_flat(), os.path.join(d, "m.pt"))
        b.load_state_dict_flat(torch.load(os.path.join(d, "m.pt")))
    tokens = torch.randint(0, cfg.vocab, (1, 16), generator=torch.Generator().manual_seed(1))
    assert torch.equal(a.forward_dense(tokens), b.forward_dense(tokens))


def test_zoo_covers_the_reference_model_table():
    """opt_125m … opt_30b and llama2_7b/13b/70b (experiments/serving/common_gpt_hyper_params.h:10-131)."""
    for n in ["opt_125m", "opt_1.3b", "opt_2.7b", "opt_6.7b", "opt_13b", "opt_30b", "llama2_7b", "llama2_13b", "llama2_70b"]:
        c = MODEL_ZOO[n]
        assert c.heads * c.head_dim == c.hidden, n
        assert c.arch == ("opt" if n.startswith("opt") else "llama")
    assert MODEL_ZOO["llama2_70b"].kv_heads == 8 and MODEL_ZOO["opt_13b"].ffn == 4 * MODEL_ZOO["opt_13b"].hidden


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _tp_worker(rank, world, port, name, ckpt, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    cfg = MODEL_ZOO[name]
    net = LlamaShard(cfg, rank, world, dist.group.WORLD, device="cpu", dtype=torch.float32, seed=77)
    net.load_hf_state_dict(torch.load(ckpt))
    tokens = torch.randint(0, cfg.vocab, (2, 24), generator=torch.Generator().manual_seed(8))
    torch.save(net.forward_dense(tokens), os.path.join(out_dir, f"r{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("name", ["tiny", "tiny_opt"])
def test_two_tensor_parallel_shards_equal_the_unsharded_model(name):
    cfg = MODEL_ZOO[name]
    full = LlamaShard(cfg, device="cpu", dtype=torch.float32, seed=4)
    _randomise(full, 3)
    tokens = torch.randint(0, cfg.vocab, (2, 24), generator=torch.Generator().manual_seed(8))
    want = full.forward_dense(tokens)
    with tempfile.TemporaryDirectory() as d:
        ckpt = os.path.join(d, "full.pt")
        torch.save(full.export_hf_state_dict(), ckpt)
        mp.spawn(_tp_worker, args=(2, _free_port(), name, ckpt, d), nprocs=2, join=True)
        outs = [torch.load(os.path.join(d, f"r{r}.pt")) for r in range(2)]
    for o in outs:
        assert (o - want).abs().max() < 1e-4 * max(1.0, want.abs().max().item())


def test_checkpoint_files_and_directories_load(tmp_path):
    from fuselink_b200.models.llama import load_checkpoint_file
    cfg = MODEL_ZOO["tiny_gpt2"]
    a = LlamaShard(cfg, device="cpu", dtype=torch.float32, seed=1)
    sd = a.export_hf_state_dict()
    keys = sorted(sd)
    torch.save({k: sd[k] for k in keys[: len(keys) // 2]}, tmp_path / "part-0.bin")
    try:
        from safetensors.torch import save_file
        save_file({k: sd[k].contiguous() for k in keys[len(keys) // 2:] if k != "lm_head.weight"}, str(tmp_path / "part-1.safetensors"))
    except ImportError:
        torch.save({k: sd[k] for k in keys[len(keys) // 2:]}, tmp_path / "part-1.pt")
    b = LlamaShard(cfg, device="cpu", dtype=torch.float32, seed=2)
    b.load_hf_state_dict(load_checkpoint_file(str(tmp_path)))
    tokens = torch.randint(0, cfg.vocab, (1, 12), generator=torch.Generator().manual_seed(1))
    assert torch.equal(a.forward_dense(tokens), b.forward_dense(tokens))
