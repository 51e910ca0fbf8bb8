#!/usr/bin/env python3
"""Headline benchmark: gpt-oss-20b-architecture MXFP4 greedy decode, tokens/s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--batch B] [--repeats R]
                    [--workload gptoss|gptoss120b|qwen2|prefill] [--exchange peer|nccl]
                    [--step persistent|per-op] [--experts block-scaled|cuda-core] [--layers L] [--synthetic-kv]

Default workload (benchmark config 3 at batch 32): 24 layers, hidden 2880, 64 q / 8 kv heads of 64, sliding window 128
alternating with full attention, sinks, 32 MXFP4 experts top-4, vocab 201088; random-init weights generated on the
device from a seed; 32 sequences with 2048-token random prompts fed token by token (as the reference feeds prompts,
lean/algorithms/Qwen2Common.lean:1446-1457), then K greedy tokens per sequence are timed.  A step = one decode step of
every sequence = one CUDA graph of the batched kernels (dense layers and MXFP4 experts on the tcgen05 tensor cores).

value   tokens/s with the argmax fed back on the device (stage `decode`), timed with CUDA events on the launching
        stream; the K-step loop runs R times over the same K positions, the line reports the median repeat.
e2e     the same metric through Base.execute_into(`infer`) once per step with host buffers: 8 bytes in, 4 bytes out
        per sequence, wall clock.
N > 1   one process per GPU (torchrun), ONE model sharded over the N GPUs: every rank holds B / N sequences (their KV
        caches, attention data parallel) and E / N experts; per layer the normalised rows go to every rank and the
        experts' partial sums back to the sequences' owners, as NVLink stores from the producing kernels (--exchange
        peer) or as NCCL all-gather + all-to-all inside the graph (--exchange nccl).  The work is fixed as N grows
        ("scaling": "strong"); value = all sequences' tokens over the slowest rank's time.
batch1  at N = 1 the line also carries benchmark config 3 at batch 1 on the same GPU (`"batch1"`: the persistent
        cooperative kernel, with its own value, e2e, roofline and phase stamps); `--batch 1` runs only that (a replica
        per GPU under torchrun; --step / --experts select its variants), `--no-batch1` leaves it out.

Other workloads (same JSON line): `gptoss120b` = benchmark config 4 (36 layers, 128 experts, 256 sequences, 4096-token
contexts on a seeded synthetic KV cache), `qwen2` = config 1 (Qwen2-0.5B, f32), `prefill` = config 2 (one MoE layer
over 2048 tokens on the tcgen05 tensor cores; under torchrun expert-parallel with one NCCL all-reduce).
`--impl reference`: the C port of the reference's CPU path (oracle/model_oracle.c) timed on the host cores on real
decode steps of the same model.
"""
from __future__ import annotations

import argparse
import json
import os
import struct
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "gpt-oss-20b MXFP4 decode tok/s"
UNIT = "tokens/s"
PROMPT = 2048


def measured_peak_gbs():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons during the timed region."""

    def __init__(self, index: int):
        self.index = index
        self.samples = []
        self.reasons = set()
        self.proc = None
        self.thread = None

    def start(self):
        q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.proc.stdout:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 6:
                continue
            try:
                self.samples.append((float(f[0]), float(f[1])))
            except ValueError:
                continue
            for n, v in zip(names, f[2:6]):
                if v.lower().startswith("active"):
                    self.reasons.add(n)

    def mark(self, timeout: float = 3.0):
        """Call right before the timed region: waits until nvidia-smi delivers (it takes a few
        100 ms to start) and drops what it reported before this point."""
        t0 = time.perf_counter()
        while self.thread and not self.samples and time.perf_counter() - t0 < timeout:
            time.sleep(0.01)
        self.first = len(self.samples)

    def stop(self):
        # a region shorter than the sampling period: wait for the sample that covers its end
        t0 = time.perf_counter()
        while self.thread and len(self.samples) <= getattr(self, "first", 0) and time.perf_counter() - t0 < 0.25:
            time.sleep(0.01)
        self.samples = self.samples[getattr(self, "first", 0):] or self.samples[-1:]
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                pass
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": sorted(self.reasons)}
        sm = sorted(s[0] for s in self.samples)
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": max(s[1] for s in self.samples),
                "reasons": sorted(self.reasons)}


def _ocfg(cfg, layers: int, max_seq: int):
    from oracle import gptoss_oracle as go
    return go.Cfg(layers=layers, hidden=cfg.hidden, inter=cfg.inter, experts=cfg.experts, top_k=cfg.top_k, n_q=cfg.n_q,
                  n_kv=cfg.n_kv, vocab=cfg.vocab, window=cfg.window, max_seq=max_seq, batch=1,
                  rope_theta=cfg.rope_theta, eps=cfg.eps, alpha=cfg.alpha, limit=cfg.limit, seed=cfg.seed)


def host_threads() -> int:
    """All host cores this process may use (torchrun exports OMP_NUM_THREADS=1; the C oracle is given the count)."""
    return len(os.sched_getaffinity(0))


def cpu_pieces(cfg, ctx: int, threads: int, reps: int = 3):
    """Decode steps of a 2-layer model of the workload's widths (one sliding and one full-attention layer, the
    whole vocabulary) on the C oracle, at context `ctx` on a synthetic KV cache: seconds per layer and for the
    final norm + lm_head + argmax, measured per piece inside real steps (oracle/model_oracle.c keeps the split)."""
    from oracle import c_oracle
    o = c_oracle.GptOssC(_ocfg(cfg, 2, ctx + reps + 2), threads=threads)
    o.fill_kv()
    o.step(1, ctx)                                     # warm-up
    s0 = o.stats()
    for i in range(reps):
        o.step(1 + i, ctx + 1 + i)
    s1 = o.stats()
    o.close()
    layer_s = sum(s1[k] - s0[k] for k in ("dense_s", "attention_s", "moe_s")) / (2 * reps)
    head_s = (s1["head_s"] - s0["head_s"]) / reps
    return layer_s, head_s


def cpu_baseline(cfg, ctx: int):
    """The GPU arm's reported CPU baseline: the C port (oracle/model_oracle.c: the reference's RowDotBench GEMV
    fold, its MX block dot, RMSNorm, RoPE, attention, argmax) on a bounded sample, a 2-layer model of the
    workload's widths with the full vocabulary, timed on all host threads and on one (the reference's CPU GEMV is
    single-threaded).  A whole step is composed from the measured pieces: layers x per-layer time + head time."""
    threads = host_threads()
    layer_all, head_all = cpu_pieces(cfg, ctx, threads, reps=3)
    layer_1, head_1 = cpu_pieces(cfg, ctx, 1, reps=1)
    step_all = cfg.layers * layer_all + head_all
    step_1 = cfg.layers * layer_1 + head_1
    return {"value": 1.0 / step_all, "unit": UNIT, "cores": threads, "kind": "port",
            "one_core": {"value": 1.0 / step_1, "cores": 1, "ms_per_step": step_1 * 1e3},
            "ms_per_step": step_all * 1e3, "nproc": os.cpu_count(),
            "sample": f"real decode steps of a 2-layer model of the workload's widths (full vocabulary, context {ctx}, "
                      f"synthetic KV cache): {layer_all * 1e3:.1f} ms per layer and {head_all * 1e3:.1f} ms for norm + "
                      f"lm_head + argmax on {threads} threads ({layer_1 * 1e3:.0f} and {head_1 * 1e3:.0f} ms on one); "
                      f"a step = {cfg.layers} x layer + head"}


def cpu_reference(cfg, ctx: int, steps: int, warmup: int, budget_s: float = 150.0):
    """The reference arm: REAL decode steps of the whole 24-layer workload on the C port, all host threads, at
    context `ctx` on a synthetic KV cache (the 2048-token prompt is not replayed on the CPU).  Runs up to `steps`
    timed steps after `warmup`, fewer when the time budget runs out (said in `sample`).  Falls back to composing
    the step from measured pieces when the host cannot hold the 14 GB of weights."""
    from oracle import c_oracle
    threads = host_threads()
    t_build = time.perf_counter()
    try:
        o = c_oracle.GptOssC(_ocfg(cfg, cfg.layers, ctx + steps + warmup + 2), threads=threads)
    except MemoryError:
        base = cpu_baseline(cfg, ctx)
        base["sample"] = "host memory too small for the whole model; " + base["sample"]
        return base, 1.0 / base["value"], 0
    o.fill_kv()
    t_build = time.perf_counter() - t_build
    tok, pos, times = 1, ctx, []
    t_start = time.perf_counter()
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        tok = o.step(tok, pos)
        dt = time.perf_counter() - t0
        pos += 1
        if i >= min(warmup, 1):
            times.append(dt)
        if time.perf_counter() - t_start > budget_s and len(times) >= 2:
            break
    st = o.stats()
    o.close()
    layer_1, head_1 = cpu_pieces(cfg, ctx, 1, reps=1)
    step_1 = cfg.layers * layer_1 + head_1
    t_step = float(np.median(times))
    total = st["dense_s"] + st["attention_s"] + st["moe_s"] + st["head_s"]
    base = {"value": 1.0 / t_step, "unit": UNIT, "cores": threads, "kind": "port", "nproc": os.cpu_count(),
            "ms_per_step": t_step * 1e3, "steps_timed": len(times),
            "one_core": {"value": 1.0 / step_1, "cores": 1, "ms_per_step": step_1 * 1e3,
                         "sample": "composed from a 2-layer model's measured per-layer and head times on one thread"},
            "share": {k: round(st[k + "_s"] / total, 3) for k in ("dense", "attention", "moe", "head")},
            "sample": f"{len(times)} real decode steps of the whole {cfg.layers}-layer model (weights generated from the "
                      f"seed in {t_build:.0f} s, synthetic KV cache at context {ctx}), median {t_step * 1e3:.0f} ms, "
                      f"min {min(times) * 1e3:.0f}, max {max(times) * 1e3:.0f}, on {threads} threads"}
    return base, t_step, len(times)


def f32_to_bf16_values(x: np.ndarray) -> np.ndarray:
    """x rounded to bf16 (nearest even), as f32 values."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    r = ((u + np.uint64(0x7FFF) + ((u >> np.uint64(16)) & np.uint64(1))) >> np.uint64(16)).astype(np.uint32) << np.uint32(16)
    return r.view(np.float32).reshape(x.shape)


def run_qwen2(a, rank: int):
    """benchmark config 1: Qwen2-0.5B shapes, f32 weights and cache, 32-token prompt fed
    token by token, K greedy tokens; single GPU by definition (rank 0 only)."""
    if rank != 0:
        return
    from base_b200.qwen2 import QWEN2_0_5B, Qwen2
    import dataclasses
    prompt_len = 32
    cfg = dataclasses.replace(QWEN2_0_5B, max_seq=prompt_len + a.warmup + 2 * a.steps + 8)
    m = Qwen2(cfg)
    rng = np.random.default_rng(1000 * 1)
    prompt = rng.integers(0, cfg.vocab, size=prompt_len)
    tok = 0
    for pos in range(prompt_len):
        tok = int(m.infer([int(prompt[pos])], [pos])[0])
    pos = prompt_len
    m.prep([tok], [pos])
    if a.warmup:
        w = m.decode(a.warmup)
        tok, pos = int(w[-1, 0]), pos + a.warmup
    sampler = ClockSampler(0)
    sampler.start()
    sampler.mark()
    m.prep([tok], [pos])
    toks, ms = m.decode(a.steps, timed=True)
    tok2, pos2 = int(toks[-1, 0]), pos + a.steps
    t0 = time.perf_counter()
    for i in range(a.steps):
        tok2 = int(m.infer([tok2], [pos2 + i])[0])
    e2e_s = time.perf_counter() - t0
    clocks = sampler.stop()
    m.close()
    peak, peak_kind = measured_peak_gbs()
    step_bytes = cfg.step_bytes(pos + a.steps // 2)
    step_s = ms * 1e-3 / a.steps
    launches = a.steps * (1 + cfg.layers * 5 + 2)
    line = {"metric": "qwen2-0.5b f32 decode tok/s", "value": a.steps / (ms * 1e-3), "unit": UNIT, "n_gpus": 1,
            "steps": a.steps, "warmup": a.warmup, "ms_per_step": ms / a.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "Qwen2-0.5B decode, f32, batch 1, 32-token prompt, greedy (benchmark config 1)",
                       "layers": cfg.layers, "hidden": cfg.hidden, "vocab": cfg.vocab, "context": prompt_len,
                       "step": "one launch per operation (CUDA graph)",
                       "l2": "each step streams ~2 GB of weights, far larger than L2; no flush needed"},
            "e2e": {"value": a.steps / e2e_s, "unit": UNIT, "h2d_bytes_per_step": 8, "d2h_bytes_per_step": 8},
            "gpu_launches": launches, "clocks": clocks,
            # the step as a whole against the HBM roofline (its GEMVs are 99.9 % of the bytes)
            "roofline": {"kernel": "whole step (gemv_fused dominates)", "bound": "hbm",
                         "achieved": step_bytes / step_s / 1e9, "peak": peak, "unit": "GB/s",
                         "frac": step_bytes / step_s / 1e9 / peak, "peak_source": peak_kind, "traffic": None,
                         "bytes_per_launch": step_bytes, "us_per_launch": step_s * 1e6}}
    emit_line(line)


def run_prefill(a, rank: int):
    """benchmark config 2: one gpt-oss-20b MoE layer over 2048 tokens (bf16 x, router skew
    ~N(0,0.5) so the experts get uneven token counts), grouped GEMMs on the tcgen05 tensor
    cores.  A step = the whole layer (bf16 conversion, router, top-k, routing tables, gate_up,
    down, combine) once.  Under torchrun (N > 1) the layer is expert-parallel: rank r owns
    E / N experts, every rank routes all tokens, and one NCCL all-reduce adds the partial
    outputs (strong scaling: the work is fixed)."""
    from base_b200.dist import Ranks
    from base_b200.moe import MoeConfig, MoeFfn, MoeFfnEP, make_moe_params, PDL, TENSOR_CORES
    world = int(os.environ.get("WORLD_SIZE", "1"))
    T = 2048
    cfg = MoeConfig()
    p = make_moe_params(cfg, seed=2000, skew=0.5)
    x = np.random.default_rng(2001).standard_normal((T, cfg.hidden)).astype(np.float32)
    x = f32_to_bf16_values(x)
    A = T * cfg.top_k
    flops = A * 2.0 * (2 * cfg.inter + cfg.hidden) * cfg.hidden
    peak, kind = 1590.0, "fallback"
    pj = ROOT / "MEASURED_PEAKS.json"
    if pj.exists():
        try:
            peak, kind = float(json.loads(pj.read_text())["bf16_tflops"]), "measured"
        except Exception:
            pass
    config = {"workload": "one gpt-oss-20b MoE FFN layer, 2048 tokens, top-4 of 32 experts, router skew 0.5 (benchmark config 2)",
              "tokens": T, "assignments": A,
              "l2": "the layer reads 424 MB of expert weights per step, larger than L2; no flush needed"}
    if world > 1:
        import torch
        ranks = Ranks("nccl")
        m = MoeFfnEP(cfg, p, ranks, max_tokens=T)
        y = m.forward(x)
        for _ in range(max(3, a.warmup)):
            m.forward(x, fetch=False)
        sampler = ClockSampler(ranks.local)
        sampler.start()
        sampler.mark()
        torch.cuda.synchronize()
        ranks.barrier()
        t0 = time.perf_counter()
        for _ in range(a.steps):
            m.local.infer(fetch=False)                 # this rank's experts (syncs the library's stream)
            m.local.export_y(m._buf.data_ptr())
            ranks.all_reduce_sum(m._buf)               # NCCL, partial sums -> layer output on every rank
        torch.cuda.synchronize()
        ranks.barrier()
        step_s = ranks.max(time.perf_counter() - t0) / a.steps
        clocks = sampler.stop()
        m.close()
        config["parallelism"] = f"expert parallel x{world}: {cfg.experts // world} experts per GPU, all-reduce of [T, hidden] f32"
        config["timing"] = "wall clock around synchronised steps, max over ranks (two streams: the library's and NCCL's)"
        line = {"metric": "gpt-oss-20b MoE layer prefill tok/s", "value": T / step_s, "unit": UNIT, "n_gpus": world,
                "steps": a.steps, "warmup": max(3, a.warmup), "ms_per_step": step_s * 1e3, "higher_is_better": True,
                "scaling": "strong", "vs_baseline": None,
                "dtype": "mxfp4 weights dequantised to bf16 in the SM, bf16 activations, f32 accumulate",
                "data": "synthetic", "config": config,
                "e2e": {"value": T / step_s, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                "gpu_launches": a.steps * 7, "clocks": clocks,
                "roofline": {"kernel": "moe_prefill_gate_up + moe_prefill_down (tcgen05)", "bound": "tensor",
                             "achieved": flops / step_s / 1e12 / world, "peak": peak, "unit": "TFLOP/s per GPU",
                             "frac": flops / step_s / 1e12 / world / peak, "peak_source": kind, "traffic": None},
                "finite": bool(np.isfinite(y).all())}
        if ranks.rank == 0:
            emit_line(line)
        ranks.close()
        return
    if rank != 0:
        return
    m = MoeFfn(cfg, p, max_tokens=T, flags=PDL | TENSOR_CORES)
    t0 = time.perf_counter()
    y = m.forward(x)                       # host buffers in and out: the end-to-end call
    e2e_first = time.perf_counter() - t0
    counts = m.route()["count"]
    for _ in range(max(3, a.warmup)):
        m.stack(1)
    sampler = ClockSampler(0)
    sampler.start()
    sampler.mark()
    ms = m.stack(a.steps, timed=True)
    t0 = time.perf_counter()
    for _ in range(4):
        m.forward(x)
    e2e_s = (time.perf_counter() - t0) / 4
    clocks = sampler.stop()
    m.close()
    step_s = ms * 1e-3 / a.steps
    config["tokens_per_expert_min_max"] = [int(counts.min()), int(counts.max())]
    line = {"metric": "gpt-oss-20b MoE layer prefill tok/s", "value": T / step_s, "unit": UNIT, "n_gpus": 1,
            "steps": a.steps, "warmup": max(3, a.warmup), "ms_per_step": ms / a.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None,
            "dtype": "mxfp4 weights dequantised to bf16 in the SM, bf16 activations, f32 accumulate",
            "data": "synthetic", "config": config,
            "e2e": {"value": T / e2e_s, "unit": UNIT, "h2d_bytes_per_step": T * cfg.hidden * 4,
                    "d2h_bytes_per_step": T * cfg.hidden * 4, "first_call_s": e2e_first},
            "gpu_launches": a.steps * 7, "clocks": clocks,
            # the two grouped GEMMs dominate; their flops over the whole layer's time
            "roofline": {"kernel": "moe_prefill_gate_up + moe_prefill_down (tcgen05)", "bound": "tensor",
                         "achieved": flops / step_s / 1e12, "peak": peak, "unit": "TFLOP/s",
                         "frac": flops / step_s / 1e12 / peak, "peak_source": kind, "traffic": None,
                         "flops_per_launch": flops, "us_per_launch": step_s * 1e6},
            "finite": bool(np.isfinite(y).all())}
    emit_line(line)


_REAL_STDOUT = None


def quiet_stdout():
    """Libraries under this process (NCCL prints its version line) write to file descriptor 1; the contract is ONE JSON
    line on stdout.  Point descriptor 1 at stderr for the run and keep the real one for `emit_line`."""
    global _REAL_STDOUT
    if _REAL_STDOUT is None:
        sys.stdout.flush()
        _REAL_STDOUT = os.fdopen(os.dup(1), "w")
        os.dup2(2, 1)


def emit_line(line: dict) -> None:
    out = _REAL_STDOUT or sys.stdout
    out.write(json.dumps(line) + "\n")
    out.flush()


def main():
    quiet_stdout()
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--prompt", type=int, default=PROMPT)
    ap.add_argument("--batch", type=int, default=32,
                    help="sequences decoded together, over all GPUs (default 32: benchmark config 3 at batch 32, sharded over "
                         "the GPUs: strong scaling).  1 = the batch-1 persistent step kernel, a full replica per GPU")
    ap.add_argument("--no-batch1", action="store_true",
                    help="with --batch > 1 on one GPU: do not also measure the batch-1 persistent kernel")
    ap.add_argument("--repeats", type=int, default=5,
                    help="how many times the K-step timed loop runs; the line reports the median repeat and the spread")
    ap.add_argument("--layers", type=int, default=0,
                    help="profiling only: a model with this many layers (a small case for ncu); the line says so in config")
    ap.add_argument("--synthetic-kv", action="store_true",
                    help="batched workloads: start from a seeded synthetic KV cache at the prompt length instead of feeding the prompt")
    ap.add_argument("--workload", choices=("gptoss", "gptoss120b", "qwen2", "prefill"), default="gptoss",
                    help="gptoss: benchmark config 3 (the headline); qwen2: benchmark config 1 (Qwen2-0.5B f32, single GPU); "
                         "prefill: benchmark config 2 (one MoE layer, 2048 tokens, tensor cores)")
    ap.add_argument("--exchange", choices=("peer", "nccl"), default="peer",
                    help="N > 1: the step's dispatch and combine as stores into peer memory by the kernels themselves, or NCCL")
    ap.add_argument("--step", choices=("persistent", "per-op"), default="persistent",
                    help="one persistent kernel per decode step (default) or one launch per operation")
    ap.add_argument("--experts", choices=("block-scaled", "cuda-core"), default="block-scaled",
                    help="with --step persistent: the expert phases on the block-scaled tensor cores (tcgen05.mma "
                         "kind::mxf4, default) or on CUDA cores + legacy MMA")
    a = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))

    if a.workload == "qwen2":
        return run_qwen2(a, rank)
    if a.workload == "prefill":
        return run_prefill(a, rank)
    if a.workload == "gptoss120b":
        # benchmark config 4: gpt-oss-120b shapes (36 layers, 128 experts), batch 256, KV context 4096 (synthetic cache)
        if a.batch == 32:
            a.batch = 256
        if a.prompt == PROMPT:
            a.prompt = 4096
        a.synthetic_kv = True
        return run_batched(a, rank, world, local)
    if a.batch > 1:
        return run_batched(a, rank, world, local)
    return run_batch1(a, rank, world, local)


def run_batch1(a, rank: int, world: int, local: int, ranks=None, emit: bool = True):
    """benchmark config 3 at batch 1 per GPU: the persistent step kernel (or the per-operation graph); under
    torchrun every rank decodes its own sequence on a full replica (weak scaling, no data-path collective)."""
    from base_b200.gptoss import GPT_OSS_20B, GptOss, PDL, PERSISTENT, BLOCK_SCALED
    import dataclasses
    mx = a.step == "persistent" and a.experts == "block-scaled"
    cfg = dataclasses.replace(GPT_OSS_20B, max_seq=a.prompt + a.warmup + 2 * a.steps + 8,
                              flags=PDL | (PERSISTENT if a.step == "persistent" else 0) | (BLOCK_SCALED if mx else 0))
    if a.layers:
        cfg = dataclasses.replace(cfg, layers=a.layers)
    config = {"workload": "gpt-oss-20b decode, batch 1 per GPU, 2048-token prompt, greedy (benchmark config 3)",
              "layers": cfg.layers, "hidden": cfg.hidden, "experts": cfg.experts, "top_k": cfg.top_k,
              "vocab": cfg.vocab, "context": a.prompt, "batch_per_gpu": 1,
              "parallelism": f"replicas x{a.gpus}" if a.gpus > 1 else "single GPU",
              "step": "one persistent cooperative kernel" if a.step == "persistent" else "one launch per operation (CUDA graph)",
              "l2": "each step streams ~3.7 GB of weights, far larger than L2; no flush needed"}
    if a.step == "persistent":
        config["expert_phases"] = ("block-scaled tensor cores (tcgen05.mma kind::mxf4)" if mx else
                             "CUDA cores + legacy MMA dequantisation")

    if a.impl == "reference":
        if rank != 0:
            return
        base, t_step, n_timed = cpu_reference(cfg, a.prompt, a.steps, a.warmup)
        config = dict(config, step="C port of the reference's CPU path, one decode step per call",
                      parallelism=f"{base['cores']} host threads")
        config.pop("expert_phases", None)
        line = {"metric": METRIC, "value": base["value"], "unit": UNIT, "n_gpus": a.gpus, "steps": a.steps,
                "steps_timed": n_timed, "warmup": a.warmup, "ms_per_step": t_step * 1e3, "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "mxfp4 weights, f32 accumulate", "data": "synthetic",
                "config": config, "impl": "reference", "cpu_baseline": base,
                "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        emit_line(line)
        return

    from base_b200.dist import Ranks
    own_ranks = ranks is None
    if own_ranks:
        ranks = Ranks("nccl" if world > 1 else None)
    barrier, max_over_ranks = ranks.barrier, ranks.max

    rng0 = np.random.default_rng(1000 * 3 + rank)
    first_tok = int(rng0.integers(0, cfg.vocab))
    try:
        m = GptOss(cfg)
        m.infer([first_tok], [0])             # the first launch is where a cooperative grid that does not fit is refused
    except RuntimeError as err:
        if a.step != "persistent":
            raise
        # the cooperative launch needs every SM of the device for one CTA each; where that is not
        # available (a partitioned or shared device) fall back to the per-operation graph and say so
        print(f"bench: persistent step kernel unavailable ({err}); using the per-operation graph", file=sys.stderr)
        cfg = dataclasses.replace(cfg, flags=PDL)
        config["step"] = "one launch per operation (CUDA graph); persistent kernel unavailable on this device"
        m = GptOss(cfg)
    rng = np.random.default_rng(1000 * 3 + rank)
    prompt = rng.integers(0, cfg.vocab, size=a.prompt)
    tok = 0
    for pos in range(a.prompt):
        tok = int(m.infer([int(prompt[pos])], [pos])[0])
    pos = a.prompt
    # warm-up steps (untimed), device feedback
    m.prep([tok], [pos])
    if a.warmup:
        w = m.decode(a.warmup)
        tok, pos = int(w[-1, 0]), pos + a.warmup

    sampler = ClockSampler(local)
    sampler.start()
    sampler.mark()
    # the K-step loop, `repeats` times: every repeat generates the SAME K positions after the prompt (the KV rows it
    # wrote are overwritten by the next), so the repeats are the same work; each is timed by device events and
    # reduced to the max over ranks; the line reports the median repeat
    rep_ms = []
    for _ in range(max(1, a.repeats)):
        barrier()
        m.prep([tok], [pos])
        toks, ms_r = m.decode(a.steps, timed=True)
        barrier()
        rep_ms.append(max_over_ranks(ms_r))
    order = sorted(range(len(rep_ms)), key=lambda i: rep_ms[i])
    mid = order[len(order) // 2]
    ms = rep_ms[mid]
    pos_mid = pos
    value = world * a.steps / (ms * 1e-3)

    # end to end: one execute_into per token, host buffers in and out
    # the same K positions once more
    tok2, pos2 = tok, pos
    barrier()
    t0 = time.perf_counter()
    seq = []
    for i in range(a.steps):
        tok2 = int(m.infer([tok2], [pos2 + i])[0])
        seq.append(tok2)
    e2e_s = max_over_ranks(time.perf_counter() - t0)
    barrier()
    clocks = sampler.stop()

    peak, peak_kind = measured_peak_gbs()
    persistent = bool(cfg.flags & PERSISTENT)
    step_bytes = cfg.step_bytes(pos_mid + a.steps // 2)
    step_s = ms * 1e-3 / a.steps
    gu_bytes, dn_bytes = cfg.gate_up_bytes(cfg.top_k), cfg.down_bytes(cfg.top_k)
    if persistent:
        # The step is ONE kernel (mega_decode): its launch duration is the step
        # time measured above with device events; its algorithmic bytes are the
        # weights and cache rows one step touches.  The phase stamps the kernel
        # leaves give the expert GEMVs' own share.
        ph = m.phase_times(m.trace_ctas())
        gu_us = ph["gate_up_first_tile"] + ph["gate_up"]
        dn_us = ph["down_first_tile"] + ph["down"]
        achieved = step_bytes / step_s / 1e9
        roof = {"kernel": "mega_decode", "bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                "frac": achieved / peak, "peak_source": peak_kind,
                # DRAM bytes per launch: an ncu capture of a 2-layer model of the same widths moved
                # 1.023 (block-scaled experts) or 1.018 x its algorithmic bytes (summary under profiles/); scaled by bytes
                "traffic": (1.023 if cfg.flags & 64 else 1.018) * step_bytes,
                "bytes_per_launch": step_bytes, "us_per_launch": step_s * 1e6,
                "phases_us_per_layer": {k: round(v, 2) for k, v in ph.items()},
                "expert_gemv": {"gate_up_gbs": gu_bytes / (gu_us * 1e-6) / 1e9, "gate_up_us": gu_us,
                                "down_gbs": dn_bytes / (dn_us * 1e-6) / 1e9, "down_us": dn_us,
                                "frac_of_peak": (gu_bytes + dn_bytes) / ((gu_us + dn_us) * 1e-6) / 1e9 / peak}}
        launches = a.steps * len(rep_ms)
    else:
        # one launch per operation: the step as a whole against the HBM roofline (its expert GEMVs
        # dominate; their own numbers are in profiles/moe_gate_up_config0_ncu_full.md)
        achieved = step_bytes / step_s / 1e9
        roof = {"kernel": "whole step (moe_gate_up_stream dominates)", "bound": "hbm", "achieved": achieved, "peak": peak,
                "unit": "GB/s", "frac": achieved / peak, "peak_source": peak_kind, "traffic": None,
                "bytes_per_launch": step_bytes, "us_per_launch": step_s * 1e6}
        launches = a.steps * len(rep_ms) * (1 + cfg.layers * 6 + 2)
    line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": a.gpus, "steps": a.steps, "warmup": a.warmup,
            "ms_per_step": ms / a.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "mxfp4 experts / bf16 dense weights, f32 accumulate", "data": "synthetic",
            "config": config,
            "e2e": {"value": world * a.steps / e2e_s, "unit": UNIT, "h2d_bytes_per_step": 8, "d2h_bytes_per_step": 8},
            "gpu_launches": launches, "clocks": clocks, "roofline": roof,
            "repeats": {"n": len(rep_ms), "ms_per_step": [round(r / a.steps, 5) for r in rep_ms],
                        "reported": "median", "min_tokens_per_s": world * a.steps / (max(rep_ms) * 1e-3),
                        "max_tokens_per_s": world * a.steps / (min(rep_ms) * 1e-3)}}
    m.close()
    if rank == 0 and emit:
        line["cpu_baseline"] = cpu_baseline(cfg, a.prompt)
        emit_line(line)
    if own_ranks:
        ranks.close()
    return line



def run_batched(a, rank: int, world: int, local: int):
    """benchmark config 3 at batch `--batch` (default 32): ONE model over all GPUs.  Every GPU holds batch / N of the
    sequences (their KV caches; attention and dense weights replicated) and experts / N of every layer's experts;
    per layer an all-gather of the normalised hidden states and an all-to-all of the experts' partial sums (NCCL,
    captured in the step's CUDA graph).  The work is fixed as N grows: strong scaling.  On one GPU the same
    launches run without the collectives."""
    import dataclasses
    from base_b200.gptoss import GPT_OSS_20B, GptOss, PDL, BATCHED
    from base_b200.dist import Ranks
    Bg = a.batch
    big = a.workload == "gptoss120b"
    model = dataclasses.replace(GPT_OSS_20B, layers=36, experts=128) if big else GPT_OSS_20B
    name = "gpt-oss-120b" if big else "gpt-oss-20b"
    if Bg % world or model.experts % world:
        raise SystemExit(f"--batch {Bg} and the {model.experts} experts must be divisible by the {world} GPUs")
    per = Bg // world
    reps = max(1, a.repeats)
    if a.layers:
        model = dataclasses.replace(model, layers=a.layers)
    cfg = dataclasses.replace(model, batch=per, max_seq=a.prompt + a.warmup + 2 * a.steps + 8,
                              flags=PDL | BATCHED, ep_rank=rank, ep_world=world)
    metric = METRIC.replace("gpt-oss-20b", name)
    config = {"workload": f"{name} decode, {Bg} sequences, {a.prompt}-token " +
                          ("contexts (seeded synthetic KV cache)" if a.synthetic_kv else "prompts") +
                          f", greedy (benchmark config {'4' if big else '3'}, batch {Bg})",
              "layers": cfg.layers, "hidden": cfg.hidden, "experts": cfg.experts, "top_k": cfg.top_k, "vocab": cfg.vocab,
              "context": a.prompt, "global_batch": Bg, "batch_per_gpu": per,
              "parallelism": f"expert parallel x{world}" if world > 1 else "single GPU",
              "step": "one CUDA graph per step: tcgen05 skinny GEMMs (dense), block-scaled tcgen05 expert kernel, split-KV attention",
              "l2": "each step streams >= 3.7 GB of weights per GPU, far larger than L2; no flush needed"}
    if a.impl == "reference":
        if rank != 0:
            return
        one = dataclasses.replace(model, max_seq=a.prompt + a.steps + a.warmup + 8)
        if big:        # 61 GB of expert weights: the CPU step is composed from a 2-layer model's measured pieces
            base = cpu_baseline(one, a.prompt)
            t_step, n_timed = 1.0 / base["value"], 0
        else:
            base, t_step, n_timed = cpu_reference(one, a.prompt, a.steps, a.warmup)
        base["sample"] += (f"; the reference decodes one sequence per call (no batching), so {Bg} sequences cost {Bg} such "
                           "steps and its tokens/s does not depend on the batch")
        config = dict(config, step="C port of the reference's CPU path, one sequence and one decode step per call",
                      parallelism=f"{base['cores']} host threads")
        line = {"metric": metric, "value": base["value"], "unit": UNIT, "n_gpus": a.gpus, "steps": a.steps,
                "steps_timed": n_timed, "warmup": a.warmup, "ms_per_step": t_step * 1e3 * Bg, "higher_is_better": True,
                "scaling": "strong", "vs_baseline": None, "dtype": "mxfp4 weights, f32 accumulate", "data": "synthetic",
                "config": config, "impl": "reference", "cpu_baseline": base,
                "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        emit_line(line)
        return

    ranks = Ranks("nccl" if world > 1 else None)
    barrier, max_over_ranks = ranks.barrier, ranks.max
    m = GptOss(cfg)
    exchange = m.exchange_init(ranks, a.exchange)
    if world > 1:
        how = ("dispatch and combine fused into the producing kernels as NVLink stores into the peers' memory, flag waits in the "
               "consumers" if exchange == "peer" else "NCCL all-gather + all-to-all per layer inside the graph")
        config["parallelism"] = (f"expert parallel x{world} (experts {cfg.experts // world} per GPU; {how}), sequences and "
                                 f"attention data parallel x{world}")
        config["exchange"] = exchange
    rng = np.random.default_rng(1000 * 3 + 17)
    if a.synthetic_kv:
        m.fill_kv()
        toks = rng.integers(0, cfg.vocab, size=Bg)[rank * per:(rank + 1) * per]
    else:
        prompt = rng.integers(0, cfg.vocab, size=(a.prompt, Bg))[:, rank * per:(rank + 1) * per]
        toks = None
        for pos in range(a.prompt):
            toks = m.infer(prompt[pos].tolist(), [pos] * per)
    toks, pos = [int(t) for t in toks], a.prompt
    m.prep(toks, [pos] * per)
    if a.warmup:
        w = m.decode(a.warmup)
        toks, pos = [int(t) for t in w[-1]], pos + a.warmup

    sampler = ClockSampler(local)
    sampler.start()
    sampler.mark()
    rep_ms = []
    for _ in range(reps):
        barrier()
        m.prep(toks, [pos] * per)
        out, ms_r = m.decode(a.steps, timed=True)
        barrier()
        rep_ms.append(max_over_ranks(ms_r))      # every repeat: the same K positions after the prompt
    order = sorted(range(len(rep_ms)), key=lambda i: rep_ms[i])
    mid = order[len(order) // 2]
    ms = rep_ms[mid]
    pos_mid = pos
    value = Bg * a.steps / (ms * 1e-3)

    # end to end: one execute_into per step with host buffers (tokens and positions in, next tokens out)
    barrier()
    t0 = time.perf_counter()
    for i in range(a.steps):
        toks = [int(t) for t in m.infer(toks, [pos + i] * per)]
    e2e_s = max_over_ranks(time.perf_counter() - t0)
    barrier()
    clocks = sampler.stop()

    # roofline of the dominant kernel, timed alone over every layer's weights with the last step's routing
    peak, peak_kind = measured_peak_gbs()
    lo, n_e = rank * (cfg.experts // world), cfg.experts // world
    hit = int((m.expert_counts()[lo:lo + n_e] > 0).sum())
    iters = 3
    gu_ms = min(m.bench_batch("gate_up", iters) for _ in range(3))
    dn_ms = min(m.bench_batch("down", iters) for _ in range(3))
    qkv_ms = min(m.bench_batch("qkv", iters) for _ in range(3))
    at_ms = min(m.bench_batch("attention", iters) for _ in range(3))
    op_ms = min(m.bench_batch("o_proj", iters) for _ in range(3))
    lm_ms = min(m.bench_batch("lm_head", iters) for _ in range(3))
    per_launch = lambda t: t * 1e-3 / (iters * cfg.layers)
    gu_bytes, dn_bytes = cfg.gate_up_bytes(hit), cfg.down_bytes(hit)
    qkv_bytes = (cfg.n_q + 2 * cfg.n_kv) * cfg.head_dim * cfg.hidden * 2
    step_bytes = cfg.step_bytes(pos_mid + a.steps // 2, experts_hit=hit)
    step_s = ms * 1e-3 / a.steps
    achieved = gu_bytes / per_launch(gu_ms) / 1e9
    roof = {"kernel": "moe_batch_mx_gate_up", "bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
            "frac": achieved / peak, "peak_source": peak_kind,
            # dram__bytes_read + write of one launch, from the ncu capture of this kernel on a 2-layer model of the 20b
            # widths (profiles/moe_batch_mx_gate_up_ncu_full.md): a launch there is a layer's experts, as here
            "traffic": 280925952 if (not big and world == 1 and Bg == 32) else None,
            "bytes_per_launch": gu_bytes, "us_per_launch": per_launch(gu_ms) * 1e6, "experts_hit_per_gpu": hit,
            "other_kernels": {"moe_batch_mx_down": {"gbs": dn_bytes / per_launch(dn_ms) / 1e9, "us_per_launch": per_launch(dn_ms) * 1e6},
                              "dense_tc_gemm_qkv": {"gbs": qkv_bytes / per_launch(qkv_ms) / 1e9, "us_per_launch": per_launch(qkv_ms) * 1e6},
                              "dense_tc_gemm_o_proj": {"gbs": cfg.hidden * cfg.n_q * cfg.head_dim * 2 / per_launch(op_ms) / 1e9, "us_per_launch": per_launch(op_ms) * 1e6},
                              "dense_tc_gemm_lm_head": {"gbs": cfg.vocab * cfg.hidden * 2 / (lm_ms * 1e-3 / iters) / 1e9, "us_per_launch": lm_ms * 1e3 / iters},
                              "attn_decode_batch": {"us_per_launch": per_launch(at_ms) * 1e6}},
            "whole_step": {"bytes_per_gpu": step_bytes, "achieved": step_bytes / step_s / 1e9, "frac": step_bytes / step_s / 1e9 / peak}}
    launches_per_step = m.capture()          # counted by the library from the step's own launch sequence
    line = {"metric": metric, "value": value, "unit": UNIT, "n_gpus": a.gpus, "steps": a.steps, "warmup": a.warmup,
            "ms_per_step": ms / a.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "mxfp4 experts / bf16 dense weights, f32 accumulate", "data": "synthetic", "config": config,
            "e2e": {"value": Bg * a.steps / e2e_s, "unit": UNIT, "h2d_bytes_per_step": 8 * per, "d2h_bytes_per_step": 4 * per},
            "gpu_launches": a.steps * len(rep_ms) * launches_per_step, "clocks": clocks, "roofline": roof,
            "repeats": {"n": len(rep_ms), "ms_per_step": [round(r / a.steps, 5) for r in rep_ms], "reported": "median",
                        "min_tokens_per_s": Bg * a.steps / (max(rep_ms) * 1e-3), "max_tokens_per_s": Bg * a.steps / (min(rep_ms) * 1e-3)}}
    m.exchange_close(ranks)
    m.close()
    if world == 1 and not a.no_batch1 and not big:
        # the batch-1 workload of the same config on the same GPU: the persistent step kernel
        b1 = run_batch1(a, rank, world, local, ranks=ranks, emit=False)
        line["batch1"] = {k: b1[k] for k in ("value", "ms_per_step", "e2e", "roofline", "repeats", "gpu_launches")}
        line["batch1"]["config"] = b1["config"]
    if rank == 0:
        line["cpu_baseline"] = cpu_baseline(dataclasses.replace(model), a.prompt)
        emit_line(line)
    ranks.close()


if __name__ == "__main__":
    main()
