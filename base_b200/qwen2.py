"""Host side of the `native:qwen2` stage program (benchmark config 1): config,
load header and a driver with the reference's decode protocol
(lean/algorithms/Qwen2Common.lean:30, 830-864).  Host logic only."""
from __future__ import annotations

import os
import struct
from dataclasses import dataclass

import numpy as np

from . import py_base

MAGIC = 0x31325751  # "QW21"
KIND = dict(ln1=0, wqkv=1, bqkv=2, wo=3, ln2=4, wgu=5, wdn=6, embed=16, lnf=17)


@dataclass
class Qwen2Config:
    layers: int = 24
    hidden: int = 896
    inter: int = 4864
    n_q: int = 14
    n_kv: int = 2
    head_dim: int = 64
    vocab: int = 151936
    max_seq: int = 2048
    batch: int = 1
    rope_theta: float = 1e6
    eps: float = 1e-6
    seed: int = 0
    flags: int = 1

    def header(self) -> bytes:
        h = struct.pack("<10I2f4I", MAGIC, self.layers, self.hidden, self.inter, self.n_q, self.n_kv, self.head_dim,
                        self.vocab, self.max_seq, self.batch, self.rope_theta, self.eps, self.seed, self.flags, 0, 0)
        assert len(h) == 64
        return h

    def step_bytes(self, ctx_len: int) -> int:
        """Algorithmic bytes of one decode step: every weight once (f32) + the KV read."""
        H, F = self.hidden, self.inter
        qd, kvd = self.n_q * 64, self.n_kv * 64
        per_layer = ((qd + 2 * kvd) * H + H * qd + 2 * F * H + H * F) * 4
        return self.layers * per_layer + self.vocab * H * 4 + self.layers * self.batch * ctx_len * 2 * kvd * 4


ON_DISK = 8      # header flags bit 3: one layer's weights and one K/V pair on the device, the rest on disk (open_files)

QWEN2_0_5B = Qwen2Config()


class Qwen2:
    def __init__(self, cfg: Qwen2Config):
        self.cfg = cfg
        self.art = py_base.native_artifact("qwen2")
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
        nb = n * self.cfg.batch * 4
        out = bytearray(nb + (4 if timed else 0))
        self.base.execute_into(self.art.extras["decode"], struct.pack("<I", n), out)
        toks = np.frombuffer(bytes(out[:nb]), dtype="<u4").reshape(n, self.cfg.batch)
        return (toks, struct.unpack("<f", bytes(out[nb:]))[0]) if timed else toks

    def logits(self) -> np.ndarray:
        out = bytearray(self.cfg.batch * self.cfg.vocab * 4)
        self.base.execute_into(self.art.extras["fetchLogits"], b"", out)
        return np.frombuffer(bytes(out), dtype="<f4").reshape(self.cfg.batch, self.cfg.vocab)

    def tensor(self, layer: int, kind: str, count: int) -> np.ndarray:
        out = bytearray(count * 4)
        self.base.execute_into(self.art.extras["fetchTensor"], struct.pack("<2I", layer, KIND[kind]), out)
        return np.frombuffer(bytes(out), dtype="<f4")

    def open_files(self, weights_path: str, cache_path: str) -> None:
        """ON_DISK instances: the flat f32 weight file to stream the layers from (base_b200.convert.write_qwen2_flat) and
        the file to keep the KV cache in (created here); before the first step."""
        self.base.execute(self.art.extras["openFiles"], os.fsencode(weights_path) + b"\0" + os.fsencode(cache_path) + b"\0")

    def set_tensor(self, layer: int, kind: str, values) -> None:
        """Replace a seeded tensor by real f32 weights (stage `setTensor`; layout as `tensor` returns it)."""
        a = np.ascontiguousarray(values, dtype="<f4")
        self.base.execute(self.art.extras["setTensor"], struct.pack("<2I", layer, KIND[kind]) + a.tobytes())

    def close(self):
        self.base.close()
