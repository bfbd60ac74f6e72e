"""Synthetic request traces in the format the online serving experiment replays (``ts: .. prompt: .. shared: .. out: ..``,
one request per line; reader: experiments/serving/online_model.hh:41-98).  The reference reads its traces from a file that is
not in its tree (online_test.sbatch:21) and leaves the generator as an empty placeholder
(experiments/serving/experiment/common/gen_input.py); this is that generator.

    python -m fuselink_b200.serving.tracegen --requests 200 --rate 4 --prompt-max 2048 > trace.txt

Arrivals are a Poisson process of ``rate`` requests per second; prompt lengths are uniform in [prompt_min, prompt_max], a
``shared_fraction`` of each prompt (at most) counts as an already cached prefix, output lengths are uniform in
[out_min, out_max].  The same seed gives the same trace.
"""
from __future__ import annotations

import argparse
import random
from typing import List


def generate(requests: int = 100, rate: float = 5.0, prompt_min: int = 32, prompt_max: int = 2048, shared_fraction: float = 0.25,
             out_min: int = 4, out_max: int = 64, seed: int = 0) -> List[str]:
    assert requests >= 0 and rate > 0 and 1 <= prompt_min <= prompt_max and 0 <= shared_fraction <= 1 and 1 <= out_min <= out_max
    rng, t, lines = random.Random(seed), 0.0, []
    for _ in range(requests):
        t += rng.expovariate(rate)
        prompt = rng.randint(prompt_min, prompt_max)
        shared = rng.randint(0, int(prompt * shared_fraction))
        lines.append(f"ts: {t:.4f} prompt: {prompt} shared: {shared} out: {rng.randint(out_min, out_max)}")
    return lines


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--requests", type=int, default=100)
    ap.add_argument("--rate", type=float, default=5.0, help="mean arrivals per second")
    ap.add_argument("--prompt-min", type=int, default=32)
    ap.add_argument("--prompt-max", type=int, default=2048)
    ap.add_argument("--shared-fraction", type=float, default=0.25)
    ap.add_argument("--out-min", type=int, default=4)
    ap.add_argument("--out-max", type=int, default=64)
    ap.add_argument("--seed", type=int, default=0)
    a = ap.parse_args(argv)
    print("\n".join(generate(a.requests, a.rate, a.prompt_min, a.prompt_max, a.shared_fraction, a.out_min, a.out_max, a.seed)))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
