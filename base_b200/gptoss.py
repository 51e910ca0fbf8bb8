"""Host side of the `native:gptoss` stage program: model configs, the load
header, and a driver over Base/execute_into that follows the reference's decode
protocol (lean/algorithms/Qwen2Common.lean:30, 830-864: per call
data = [token_id:u32][pos:u32], out = [next_token:u32]).  Host logic only.
"""
from __future__ import annotations

import struct
from dataclasses import dataclass, asdict

import numpy as np

from . import py_base

MAGIC = 0x31534F47  # "GOS1"
PDL, ONE_COLUMN = 1, 4
PERSISTENT = 32   # the whole decode step as one cooperative persistent kernel (batch 1)
BLOCK_SCALED = 64 # with PERSISTENT: the experts run on the block-scaled tensor cores (tcgen05.mma kind::mxf4)
BATCHED = 128     # up to 256 sequences per GPU: dense layers and experts on the tcgen05 tensor cores, every weight read
                  # once per step for all sequences; with ep_world > 1 expert-parallel over that many GPUs

KIND = dict(ln1=0, wqkv=1, bqkv=2, sinks=3, wo=4, bo=5, ln2=6, wr=7, br=8, gu_codes=9, gu_scales=10, gu_bias=11,
            dn_codes=12, dn_scales=13, dn_bias=14, embed=16, lm_head=17, lnf=18)
GLOBAL_LAYER = 1000


@dataclass
class GptOssConfig:
    layers: int = 24
    hidden: int = 2880
    inter: int = 2880
    experts: int = 32
    top_k: int = 4
    n_q: int = 64
    n_kv: int = 8
    head_dim: int = 64
    vocab: int = 201088
    window: int = 128
    max_seq: int = 2304
    batch: int = 1
    rope_theta: float = 150000.0
    eps: float = 1e-5
    alpha: float = 1.702
    limit: float = 7.0
    seed: int = 0
    flags: int = PDL
    test_skip_fill: int = 0   # failure-path test hook: 1 + the ring fill the persistent kernel's producers leave out
    test_spin: int = 0        # failure-path test hook: iteration limit of the persistent kernel's waits (0: default)
    ep_rank: int = 0          # BATCHED over several GPUs: this process's rank ...
    ep_world: int = 0         # ... of this many (0 or 1: one GPU); `batch` is the number of sequences per GPU

    def header(self) -> bytes:
        h = struct.pack("<13I4f4I4I7I", MAGIC, self.layers, self.hidden, self.inter, self.experts, self.top_k,
                        self.n_q, self.n_kv, self.head_dim, self.vocab, self.window, self.max_seq, self.batch,
                        self.rope_theta, self.eps, self.alpha, self.limit, self.seed, self.flags, 0, 0,
                        self.test_skip_fill, self.test_spin, self.ep_rank, self.ep_world, *([0] * 7))
        assert len(h) == 128
        return h

    # ---- algorithmic bytes of one decode step (every operand counted once) ----
    def expert_bytes(self) -> int:
        H, I = self.hidden, self.inter
        return 2 * I * (H // 2) + 2 * I * (H // 32) + 2 * I * 4 + H * (I // 2) + H * (I // 32) + H * 4

    def gate_up_bytes(self, experts_hit: int) -> int:
        H, I = self.hidden, self.inter
        return experts_hit * (2 * I * (H // 2) + 2 * I * (H // 32) + 2 * I * 4)

    def down_bytes(self, experts_hit: int) -> int:
        H, I = self.hidden, self.inter
        return experts_hit * (H * (I // 2) + H * (I // 32) + H * 4)

    def step_bytes(self, ctx_len: int, experts_hit: int | None = None) -> int:
        H, E = self.hidden, self.experts
        hit = experts_hit if experts_hit is not None else min(E, self.batch * self.top_k)
        qd, kvd = self.n_q * self.head_dim, self.n_kv * self.head_dim
        per_layer = hit * self.expert_bytes() + E * H * 4 + (qd + 2 * kvd) * H * 2 + H * qd * 2
        kv = 0
        for l in range(self.layers):
            vis = min(ctx_len, self.window) if (l % 2 == 0 and self.window) else ctx_len
            kv += self.batch * vis * 2 * kvd * 2
        return self.layers * per_layer + self.vocab * H * 2 + kv


GPT_OSS_20B = GptOssConfig()


class GptOss:
    """load once; `infer(tokens, positions)` = one decode step through the C-ABI."""

    def __init__(self, cfg: GptOssConfig):
        self.cfg = cfg
        self.art = py_base.native_artifact("gptoss")
        self.base = py_base.Base(self.art.setup)
        self.base.execute(self.art.main, cfg.header())

    def _meta(self, tokens, positions) -> bytes:
        t = np.atleast_1d(np.asarray(tokens, dtype="<u4"))
        p = np.atleast_1d(np.asarray(positions, dtype="<u4"))
        assert t.shape == p.shape == (self.cfg.batch,)
        return np.stack([t, p], axis=1).astype("<u4").tobytes()

    def prep(self, tokens, positions):
        self.base.execute(self.art.extras["prep"], self._meta(tokens, positions))

    def infer(self, tokens, positions) -> np.ndarray:
        out = bytearray(4 * self.cfg.batch)
        self.base.execute_into(self.art.extras["infer"], self._meta(tokens, positions), out)
        return np.frombuffer(bytes(out), dtype="<u4")

    def decode(self, n: int, timed: bool = False):
        """n steps with the argmax fed back on the device (after `prep`)."""
        nb = n * self.cfg.batch * 4
        out = bytearray(nb + (4 if timed else 0))
        self.base.execute_into(self.art.extras["decode"], struct.pack("<I", n), out)
        toks = np.frombuffer(bytes(out[:nb]), dtype="<u4").reshape(n, self.cfg.batch)
        if timed:
            return toks, struct.unpack("<f", bytes(out[nb:]))[0]
        return toks

    def comm_init(self, comm_id: bytes):
        """Join the expert-parallel communicator (BATCHED, ep_world > 1): `comm_id` is the 128-byte id rank 0 made
        with `new_comm_id()` and sent to every rank.  After construction, before the first step."""
        self.base.execute(self.art.extras["commInit"], comm_id)

    def peer_handles(self) -> bytes:
        """192 bytes: the handles of this rank's three exchange buffers (BATCHED, 2..8 ranks)."""
        out = bytearray(192)
        self.base.execute_into(self.art.extras["peerHandles"], b"", out)
        return bytes(out)

    def peer_init(self, handles) -> None:
        """`handles`: every rank's `peer_handles()` in rank order.  From here on the step's dispatch and combine are
        stores into the other ranks' memory by the kernels themselves (no NCCL call in the step); every rank calls
        it, after construction and before the first step."""
        self.base.execute(self.art.extras["peerInit"], b"".join(handles))
        self._peer = True

    def exchange_init(self, ranks, mode: str = "peer") -> str:
        """Set up the step's exchange over `ranks` (a base_b200.dist.Ranks): "peer" (kernels store to peer memory;
        falls back to NCCL when the ranks cannot map each other's memory) or "nccl".  Returns the mode in use."""
        if ranks.world < 2:
            return "none"
        if mode == "peer" and ranks.world <= 8:
            try:
                mine, why = self.peer_handles(), ""
            except RuntimeError as e:
                mine, why = b"", str(e)
            every = ranks.all_gather_bytes(mine)
            if all(len(h) == 192 for h in every):
                try:
                    self.peer_init(every)
                except RuntimeError as e:
                    why = str(e)
            else:
                why = why or "a rank could not export its buffers"
            if all(not w for w in ranks.all_gather_bytes(why.encode())):
                return "peer"
            if getattr(self, "_peer", False):
                raise RuntimeError("peer memory was mapped on this rank but not on every rank")
        self.comm_init(ranks.broadcast_bytes(GptOss.new_comm_id() if ranks.rank == 0 else None))
        return "nccl"

    def peer_trace(self) -> np.ndarray:
        """u64 [layers][8] time stamps (ns) of the last step's exchanging kernels: rows_to_peers start, router start,
        router after its wait, combine start, the next normalisation's start, after its wait."""
        out = bytearray(self.cfg.layers * 64)
        self.base.execute_into(self.art.extras["fetchPeerTrace"], b"", out)
        return np.frombuffer(bytes(out), dtype="<u8").reshape(self.cfg.layers, 8)

    def exchange_close(self, ranks) -> None:
        """Unmap the other ranks' memory and meet them, so that no rank frees a buffer another still maps.  Call on
        every rank before `close()` when `exchange_init` returned "peer" (harmless otherwise)."""
        if getattr(self, "_peer", False):
            self.base.execute(self.art.extras["peerClose"], b"")
            self._peer = False
        ranks.barrier()

    @staticmethod
    def new_comm_id() -> bytes:
        import ctypes
        from . import lib
        buf = ctypes.create_string_buffer(128)
        if lib().cl_b200_comm_unique_id(buf) != 0:
            raise RuntimeError(lib().cl_b200_last_error().decode())
        return buf.raw

    # ---- graph capture / replay and the launch ladder (the reference's `capture`, `replay*`, `runTo{k}` extras:
    # lean/algorithms/MlpCifarAlgorithm.lean:2233-2264, applications/ten-qwen/profile.py:34-36, 67-90)
    def capture(self) -> int:
        """Capture the step's CUDA graph without running it; returns the launches per step."""
        out = bytearray(4)
        self.base.execute_into(self.art.extras["capture"], b"", out)
        return struct.unpack("<I", bytes(out))[0]

    def replay(self, n: int = 1) -> float:
        """n launches of the captured graph on whatever tokens / positions the device holds; ms (device events)."""
        out = bytearray(4)
        self.base.execute_into(self.art.extras["replay"], struct.pack("<I", n), out)
        return struct.unpack("<f", bytes(out))[0]

    def run_to(self, k: int) -> float:
        """The first k launches of the step issued directly (no graph), one sync; ms (device events)."""
        out = bytearray(4)
        self.base.execute_into(self.art.extras["runTo"], struct.pack("<I", k), out)
        return struct.unpack("<f", bytes(out))[0]

    def launch_ladder(self, rungs, reps: int = 20) -> list:
        """The reference's launch-ladder profile (profile.py:67-82): time prefixes of the launch sequence and
        difference them.  Returns [(first, last, cumulative_us, bucket_us, us_per_launch)] per rung."""
        rows, prev_k, prev_t = [], 0, 0.0
        for k in rungs:
            for _ in range(3):
                self.run_to(k)
            t = min(self.run_to(k) for _ in range(reps)) * 1e3
            rows.append((prev_k, k, t, t - prev_t, (t - prev_t) / max(k - prev_k, 1)))
            prev_k, prev_t = k, t
        return rows

    STATE = dict(h1=0, xn=1, router_logits=2, topk_idx=3, topk_w=4, act=5, o=6, qkv=7, attn=8, y_part=9, route=10)

    def state(self, name: str, count: int, dtype="<f4") -> np.ndarray:
        """The first `count` elements of an intermediate buffer of the last step (stage `fetchState`)."""
        out = bytearray(count * np.dtype(dtype).itemsize)
        self.base.execute_into(self.art.extras["fetchState"], struct.pack("<I", self.STATE[name]), out)
        return np.frombuffer(bytes(out), dtype=dtype)

    def fill_kv(self):
        """Overwrite every layer's KV cache with the seeded synthetic rows (stage `fillKV`), so that a step at a
        late position has a full context without feeding the prompt."""
        self.base.execute(self.art.extras["fillKV"], b"")

    def trace(self, n_ctas: int) -> np.ndarray:
        """Phase time stamps (ns) of the last persistent step: u64 [n_ctas][512], n_ctas = SM count."""
        out = bytearray(n_ctas * 512 * 8)
        self.base.execute_into(self.art.extras["fetchTrace"], b"", out)
        return np.frombuffer(bytes(out), dtype="<u8").reshape(n_ctas, 512)

    # Stamps of the persistent step kernel, in order (mega_decode.cuh): one at the
    # start, then per layer the END of each of these intervals, then the same
    # first three for the lm_head phase.
    PHASES = ("qkv_input", "qkv", "barrier", "attention", "barrier", "o_proj", "barrier", "router_input", "router",
              "gate_up_first_tile", "gate_up", "barrier", "down_first_tile", "down", "barrier")

    def trace_ctas(self) -> int:
        """CTAs of the persistent step kernel (= SMs of the device)."""
        from . import lib
        ctx = struct.unpack_from("<Q", self.base.memory(), 0x10)[0]      # the CUDA context slot of the memory block
        return int(lib().cl_b200_sm_count(ctx))

    def phase_times(self, n_ctas: int) -> dict:
        """Mean microseconds per layer spent in each phase of the last persistent step:
        the slowest CTA for work phases, the last CTA to arrive for the barriers
        (i.e. the barrier's own latency), averaged over layers."""
        tr = self.trace(n_ctas).astype(np.int64)
        P, L = len(self.PHASES), self.cfg.layers
        n = min(1 + P * L, 512)
        L = (n - 1) // P
        d = np.diff(tr[:, :1 + P * L], axis=1).reshape(n_ctas, L, P) / 1e3
        out: dict = {}
        for j, name in enumerate(self.PHASES):
            col = d[:, :, j]
            out[name] = out.get(name, 0.0) + float((col.min(axis=0) if name == "barrier" else col.max(axis=0)).mean())
        out["layer_us"] = float((tr[:, P * L].max() - tr[:, 0].min()) / 1e3 / L)
        return out

    def logits(self) -> np.ndarray:
        out = bytearray(self.cfg.batch * self.cfg.vocab * 4)
        self.base.execute_into(self.art.extras["fetchLogits"], b"", out)
        return np.frombuffer(bytes(out), dtype="<f4").reshape(self.cfg.batch, self.cfg.vocab)

    def tensor(self, layer: int, kind: str, nbytes: int, dtype) -> np.ndarray:
        out = bytearray(nbytes)
        self.base.execute_into(self.art.extras["fetchTensor"], struct.pack("<2I", layer, KIND[kind]), out)
        return np.frombuffer(bytes(out), dtype=dtype)

    def dequant(self, layer: int, which: int, expert: int, row0: int, nrows: int) -> np.ndarray:
        K = self.cfg.hidden if which == 0 else self.cfg.inter
        out = bytearray(nrows * K * 4)
        self.base.execute_into(self.art.extras["fetchDequant"], struct.pack("<5I", layer, which, expert, row0, nrows), out)
        return np.frombuffer(bytes(out), dtype="<f4").reshape(nrows, K)

    BATCH_KERNELS = dict(gate_up=1, down=2, qkv=3, o_proj=4, attention=5, lm_head=6)

    def bench_batch(self, which: str, iters: int = 1) -> float:
        """Milliseconds (device events) for `iters` passes of one kernel of the batched step over every layer."""
        out = bytearray(4)
        self.base.execute_into(self.art.extras["benchBatch"], struct.pack("<2I", self.BATCH_KERNELS[which], iters), out)
        return struct.unpack("<f", bytes(out))[0]

    def expert_counts(self) -> np.ndarray:
        """Tokens per expert in the last layer of the last step (all experts, from the routing tables)."""
        return self.state("route", 1 + self.cfg.experts, "<i4")[1:]

    def close(self):
        self.base.close()
