"""The N > 1 plumbing of the benchmark on CPU: two gloo ranks, barrier, max of
the per-rank times, sum of the units, expert-parallel ownership."""
import os
import socket

import pytest
import torch.multiprocessing as mp

from base_b200.dist import Ranks, expert_range


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, out):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    r = Ranks(backend="gloo")
    r.barrier()
    seconds = 0.010 + 0.001 * rank          # rank 1 is the slow one
    out.put((rank, r.max(seconds), r.sum(5.0), r.throughput(5.0, seconds)))
    r.barrier()
    r.close()


def test_two_ranks_aggregate_like_the_benchmark_contract():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    got = sorted(out.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, mx, sm, thr in got:
        assert mx == pytest.approx(0.011)
        assert sm == pytest.approx(10.0)
        assert thr == pytest.approx(10.0 / 0.011)


def test_single_process_needs_no_group():
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
        os.environ.pop(k, None)
    r = Ranks()
    r.barrier()
    assert r.world == 1 and r.max(3.0) == 3.0 and r.throughput(4.0, 2.0) == 2.0
    r.close()


def test_expert_ranges_partition_the_experts():
    for experts, world in ((32, 1), (32, 2), (32, 8), (128, 8)):
        seen = []
        for rank in range(world):
            lo, n = expert_range(rank, world, experts)
            seen += list(range(lo, lo + n))
        assert seen == list(range(experts))
    with pytest.raises(ValueError):
        expert_range(0, 3, 32)


def _sum_worker(rank: int, world: int, port: int, out):
    import torch
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    r = Ranks(backend="gloo")
    t = torch.full((4, 3), float(rank + 1))
    r.all_reduce_sum(t)                      # the expert-parallel combine: partial sums add up on every rank
    out.put((rank, t.tolist()))
    r.barrier()
    r.close()


def test_partial_sums_all_reduce_on_every_rank():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_sum_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    got = [out.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for _, vals in got:
        assert vals == [[3.0] * 3] * 4


def _ep_worker(rank: int, world: int, port: int, out):
    import numpy as np
    from base_b200.dist import ep_moe_layer
    from base_b200.moe import MoeConfig, make_moe_params
    from oracle import moe_oracle as mo
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    r = Ranks(backend="gloo")
    cfg = MoeConfig(hidden=64, inter=64, experts=8, top_k=4)
    p = make_moe_params(cfg, seed=41)
    p["Wr"] *= 20
    x_all = np.random.default_rng(42).standard_normal((6, cfg.hidden)).astype(np.float32)     # 3 tokens per rank
    mine = x_all[rank * 3:(rank + 1) * 3]
    deq = {}

    def expert(e, row):
        if e not in deq:
            deq[e] = (mo.mx_dequant(p["gu_codes"][e], p["gu_scales"][e]), mo.mx_dequant(p["dn_codes"][e], p["dn_scales"][e]))
        return mo.expert_ffn(row, deq[e][0], p["gu_bias"][e], deq[e][1], p["dn_bias"][e], cfg.alpha, cfg.limit)[0]

    def route(xa):
        return mo.topk_softmax(mo.router_logits(xa, p["Wr"], p["br"]), cfg.top_k)

    y = ep_moe_layer(r, mine, cfg.experts, cfg.top_k, route, expert)
    want = mo.moe_ffn(x_all, p)[rank * 3:(rank + 1) * 3]
    lo, n = expert_range(rank, world, cfg.experts)
    handles = r.all_gather_bytes(b"handles-of-%d" % rank)          # the hand-out GptOss.exchange_init relies on
    assert handles == [b"handles-of-%d" % q for q in range(world)]
    out.put((rank, float(np.abs(y - want).max() / np.abs(want).max()), sorted(deq), (lo, n), r.broadcast_bytes(b"id-from-0" if rank == 0 else None)))
    r.barrier()
    r.close()


def test_expert_parallel_exchange_on_two_ranks_equals_the_unsharded_layer():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_ep_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    got = sorted(out.get(timeout=180) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, err, used, (lo, n), ident in got:
        assert err < 1e-6                                    # same products, summed per rank then over ranks
        assert all(lo <= e < lo + n for e in used) and used  # a rank only ever runs its own experts
        assert ident == b"id-from-0"


def test_exchange_counters_reach_their_targets_round_by_round():
    """The arithmetic of the kernels' own exchange (csrc/kernels/peer_xchg.cuh), restated on the host: every source rank
    adds one arrival per sequence and round to a counter that never resets; a consumer of round (step, layer) waits
    for ((step - 1) * layers + layer + 1) * per_round.  The target must be exactly what has arrived once the round is
    complete, and must not be reachable one arrival earlier (a consumer can then never run ahead of a producer)."""
    layers, per_round, world = 5, 3, 4
    counters = [0] * world                     # one rank's view: arrivals from every source rank
    for step in range(1, 4):                   # the step counter is bumped before the first layer: 1-based
        for layer in range(layers):
            target = ((step - 1) * layers + layer + 1) * per_round
            for src in range(world):
                for seq in range(per_round):
                    assert counters[src] - target < 0            # not yet: the wait would still be spinning
                    counters[src] += 1
            assert all(c - target >= 0 for c in counters) and all(c == target for c in counters)
    # 32-bit wrap: the comparison is on the signed difference
    wrap = lambda v: (v + 2 ** 31) % 2 ** 32 - 2 ** 31
    assert wrap((2 ** 32 + 5) % 2 ** 32 - (2 ** 32 - 3) % 2 ** 32) >= 0 and wrap((2 ** 32 - 3) - (2 ** 32 + 5)) < 0
