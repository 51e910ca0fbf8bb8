"""Run a few decode steps of a gpt-oss-shaped model and print the time per step: the small, fixed command to put under
a profiler (`ncu -k regex:<kernel> ... python -m base_b200.step_runner --layers 2`) or a launch-ladder, in the role of
the reference's profile.py (applications/gpt-oss/profile.py:67-82: load once, replay steps, time them).

Weights are generated on the device from the seed, the KV cache is filled with the seeded synthetic rows, so a step at
`--context` costs what a step after a real prompt of that length costs, without feeding the prompt.

Under torchrun (`torchrun --nproc-per-node N -m base_b200.step_runner ...`) the `--batch` sequences and the experts are
sharded over the N GPUs as in bench.py; `--trace` then prints, per rank, where a layer's time goes.
"""
from __future__ import annotations

import argparse
import dataclasses
import json
import os

import numpy as np

from .dist import Ranks
from .gptoss import BATCHED, BLOCK_SCALED, GPT_OSS_20B, PDL, PERSISTENT, GptOss


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--shapes", choices=("20b", "120b"), default="20b", help="32 or 128 experts (hidden 2880 either way)")
    ap.add_argument("--layers", type=int, default=2)
    ap.add_argument("--batch", type=int, default=32, help="sequences; 1 with --persistent runs the one-kernel step")
    ap.add_argument("--context", type=int, default=2048)
    ap.add_argument("--vocab", type=int, default=GPT_OSS_20B.vocab, help="a small vocabulary keeps a profiled process small")
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--persistent", action="store_true", help="batch 1: the persistent step kernel with block-scaled experts")
    ap.add_argument("--ladder", action="store_true", help="also print the launch ladder of one step (one GPU, batched step)")
    ap.add_argument("--exchange", choices=("peer", "nccl"), default="peer", help="under torchrun: how the sharded step exchanges rows")
    ap.add_argument("--trace", action="store_true",
                    help="under torchrun with the peer exchange: every rank prints where a layer's time goes (microseconds, "
                         "from the exchanging kernels' time stamps of the last step)")
    a = ap.parse_args()
    ranks = Ranks("nccl" if int(os.environ.get("WORLD_SIZE", "1")) > 1 else None)
    world, rank = ranks.world, ranks.rank
    model = dataclasses.replace(GPT_OSS_20B, layers=a.layers, experts=128 if a.shapes == "120b" else 32, vocab=a.vocab)
    if a.persistent:
        cfg = dataclasses.replace(model, batch=1, max_seq=a.context + a.steps + 8, flags=PDL | PERSISTENT | BLOCK_SCALED)
    else:
        cfg = dataclasses.replace(model, batch=a.batch // world, max_seq=a.context + a.steps + 8, flags=PDL | BATCHED,
                                  ep_rank=rank, ep_world=world)
    m = GptOss(cfg)
    mode = m.exchange_init(ranks, a.exchange) if world > 1 else "none"
    m.fill_kv()
    toks = np.random.default_rng(7).integers(0, cfg.vocab, size=cfg.batch * world)[rank * cfg.batch:(rank + 1) * cfg.batch]
    m.prep([int(t) for t in toks], [a.context] * cfg.batch)
    ranks.barrier()
    out, ms = m.decode(a.steps, timed=True)
    ranks.barrier()
    line = {"shapes": a.shapes, "layers": a.layers, "batch": cfg.batch * world, "context": a.context, "steps": a.steps,
            "ms_per_step": ms / a.steps, "last_tokens": [int(t) for t in out[-1][:4]]}
    if world > 1:
        line.update(rank=rank, gpus=world, exchange=mode)
    if a.trace and mode == "peer":
        # stamps per layer: 0 dispatch kernel starts, 1 router starts, 2 its wait is over, 3 combine kernel starts,
        # 4 the next normalisation starts, 5 its wait is over
        t = m.peer_trace().astype(np.int64)
        us = lambda x: round(float(np.mean(x)) / 1e3, 2)
        line["layer_us"] = {"attention_part": us(t[1:, 0] - t[:-1, 5]), "dispatch": us(t[:, 1] - t[:, 0]),
                            "dispatch_wait": us(t[:, 2] - t[:, 1]), "experts_part": us(t[:, 3] - t[:, 2]),
                            "combine": us(t[:, 4] - t[:, 3]), "combine_wait": us(t[:, 5] - t[:, 4])}
        line["layer_us"]["sum"] = round(sum(line["layer_us"].values()), 2)
    if a.ladder and not a.persistent:
        n = m.capture()
        line["launches_per_step"] = n
        line["ladder_us"] = [[first, last, round(bucket, 2)] for first, last, _, bucket, _ in m.launch_ladder(range(1, n + 1), reps=5)]
    for r in range(world):          # one line per rank, in rank order
        ranks.barrier()
        if r == rank:
            print(json.dumps(line), flush=True)
    m.exchange_close(ranks)
    m.close()
    ranks.close()


if __name__ == "__main__":
    main()
