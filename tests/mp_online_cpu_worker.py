"""Worker of tests/test_kernel_model_cpu.py::test_online_serving_between_processes: the trace-driven prefill -> decode
hand-off between two REAL processes on a machine without a GPU.  Rank 0 batches a trace and prefills, rank 1 decodes; the
paged KV cache, the header, the completion flag and the pool credits travel through a shared-memory heap with the KV entry
point modelled on the host.  Two pools are used in turn, so the prefill has to wait for the decoder's credits; the trace
ends with the empty header.  The decoder checks every generated token against the dense model on the same prompts (which
it can rebuild: the prompts come from a seeded generator and the header names the batch's shape)."""
import datetime
import os
import queue
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import torch
import torch.distributed as dist


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    assert world == 2
    dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=120))
    import cpu_kernel_model
    from fuselink_b200.models.llama import MODEL_ZOO, LlamaShard
    from fuselink_b200.parallel.symm import SymmetricHeap
    from fuselink_b200.serving.disagg import KVLink, ServeParams
    from fuselink_b200.serving.online import MAX_BATCH, OnlineDecode, OnlinePrefill, TraceReader, parse_trace
    from fuselink_b200.serving.scheduler import Scheduler
    from fuselink_b200.serving.tracegen import generate
    cfg = MODEL_ZOO["tiny"]
    steps = 3
    dtype = torch.float32 if os.environ.get("FL_ONLINE_DTYPE", "fp32") == "fp32" else torch.bfloat16
    p = ServeParams(cfg, MAX_BATCH, input_len=96, num_decoding_step=steps, dtype=dtype)
    with cpu_kernel_model.installed(single_process=False) as model:
        model.wait_limit_s = 60.0
        net = LlamaShard(cfg, device="cpu", seed=1, dtype=dtype, max_positions=p.input_len + steps + cfg.block_size)
        pool = 2 * p.batch_size * p.max_blocks_per_req * cfg.layers * net.kvh_local * cfg.block_size * cfg.head_dim * p.elem_bytes
        heap = SymmetricHeap.create(2 * pool + (32 << 20), device=-1)
        links = [KVLink(heap, p, net.kvh_local, name=f"kv{i}") for i in range(2)]
        reqs = parse_trace(generate(requests=23, rate=400.0, prompt_min=20, prompt_max=90, shared_fraction=0.3, out_min=2, out_max=6, seed=2))
        if rank == 0:
            pre = OnlinePrefill(p, net, links, dst_rank=1, seed=7)
            q = queue.Queue()
            TraceReader(reqs, q).start()
            sched = Scheduler(q, 6, p.input_len, policy="sjf", max_batch_tokens=300)
            served, finished = 0, False
            while not finished:
                batch, finished = sched.next_batch()
                if not batch:
                    continue
                st = pre.serve_batch(batch)
                bs = cfg.block_size
                pages = sum((r.active_prompt_len + bs - 1) // bs for r in batch)
                assert st.kv_bytes == pages * cfg.layers * links[0].page_elems * 2 * p.elem_bytes   # K and V: padding is never sent
                served += len(batch)
            pre.send_end()
            heap.check_status("prefill side")
            assert served == 23 and pre.batches - 1 >= 4, (served, pre.batches)            # both pools reused: credits were waited for
            print(f"ONLINE-MP-OK rank 0 served {served} requests in {pre.batches - 1} batches", flush=True)
        else:
            dec = OnlineDecode(p, net, links, src_rank=0)
            gen = torch.Generator().manual_seed(7)                # the prefill side's prompt generator, replayed
            served = batches = agree = total = 0
            while True:
                out = dec.serve_batch(steps)
                if out["batch"] == 0:
                    break
                B, S = out["batch"], out["padded_len"]
                hdr = links[(dec.batches - 1) % 2].hdr.local
                lens = hdr[4 + 32:4 + 32 + B].tolist()
                tokens = torch.randint(0, min(32000, cfg.vocab), (B, S), generator=gen)
                got = out["generated"]                            # [B, 1 + steps]
                assert got.shape == (B, 1 + steps)
                for b in range(B):
                    seq = tokens[b:b + 1, :lens[b]]
                    for t in range(1 + steps):
                        nxt = net.forward_dense(seq).argmax(-1)
                        agree += int(int(nxt) == int(got[b, t]))
                        total += 1
                        seq = torch.cat([seq, got[b, t].view(1, 1)], 1)        # follow what was generated: every step is judged on its own
                served += B
                batches += 1
            heap.check_status("decode side")
            # fp32: the paged path must reproduce the dense model exactly; bf16: near-ties of the arg-max may fall the other way
            need = 1.0 if dtype == torch.float32 else 0.9
            assert served == 23 and agree >= need * total, (served, agree, total)
            print(f"ONLINE-MP-OK rank 1 checked {served} requests against the dense model: {agree} of {total} tokens agree", flush=True)
        dist.barrier()
        heap.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
