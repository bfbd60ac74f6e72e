"""Command line of the serving experiments, with the reference's flag names (experiments/serving/main.cc:45-107,
online_main.cc:54-59):

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 -m fuselink_b200.serving \\
        --model_name llama3_8b --precision bf16 --input_len 2048 --batch_size 16 --block_size 16 \\
        --num_decoding_step 256 --tp_size 4 [--tracepath trace.txt] [--kv fuselink|nccl]

Ranks below world/2 run the context (prefill) stage, the others decode; rank r hands its KV shard to rank
r + world/2.  With ``--tracepath`` the online (trace-driven) experiment runs instead of the offline one.  On a single
process both stages run as virtual ranks on one GPU."""
from __future__ import annotations

import argparse
import os
import runpy
import sys


def main():
    ap = argparse.ArgumentParser(prog="fuselink_b200.serving")
    ap.add_argument("--model_name", default="llama3_8b")
    ap.add_argument("--model_path", default="dummy", help="'dummy' (random weights, as the reference's scripts pass) or a Hugging Face state_dict file / directory")
    ap.add_argument("--vocab_json_path", default="")
    ap.add_argument("--precision", default="bf16", choices=["bf16", "fp16", "fp32"])
    ap.add_argument("--input_len", type=int, default=2048)
    ap.add_argument("--batch_size", type=int, default=16)
    ap.add_argument("--block_size", type=int, default=16)
    ap.add_argument("--num_decoding_step", type=int, default=256)
    ap.add_argument("--tp_size", type=int, default=0, help="0: world/2")
    ap.add_argument("--tracepath", default="")
    ap.add_argument("--kv", default="fuselink", choices=["fuselink", "fuselink-nopipe", "nccl"])
    ap.add_argument("--device", default="cuda", choices=["cuda", "cpu"], help="cpu: only under a model of the device entry points (tests)")
    a = ap.parse_args()
    from fuselink_b200.models.llama import MODEL_ZOO

    if a.model_name not in MODEL_ZOO:
        raise SystemExit(f"unknown model {a.model_name}; known: {', '.join(MODEL_ZOO)}")
    MODEL_ZOO[a.model_name].block_size = a.block_size
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if a.tp_size and world > 1 and a.tp_size != world // 2:
        raise SystemExit(f"--tp_size {a.tp_size} needs {2 * a.tp_size} ranks (got {world})")
    if a.tracepath:
        sys.argv = ["run_online_serving.py", "--trace", a.tracepath, "--model", a.model_name, "--input-len", str(a.input_len),
                    "--decode-steps", str(a.num_decoding_step), "--device", a.device]
        runpy.run_path(os.path.join(root, "experiments", "run_online_serving.py"), run_name="__main__")
    else:
        sys.argv = ["serving_bench.py", "--model", a.model_name, "--kv", a.kv, "--batch", str(a.batch_size), "--input-len",
                    str(a.input_len), "--decode-steps", str(a.num_decoding_step), "--model-path", a.model_path, "--precision", a.precision, "--device", a.device] + (["--emulate"] if world == 1 else [])
        runpy.run_path(os.path.join(root, "bench", "serving_bench.py"), run_name="__main__")


if __name__ == "__main__":
    main()
