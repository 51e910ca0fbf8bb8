"""CPU oracle for Qwen2-architecture greedy decode (f32 weights).  TEST
INFRASTRUCTURE ONLY.

Follows the reference's shipped decode program op by op
(lean/algorithms/Qwen2Common.lean:1730-1749, args :1959-1997): rmsnorm
(Qwen2Proven.lean:304-333; eps of benchmark config 1 = 1e-6), q/k/v = W x + b
(:954-959), half-split RoPE on q and k from a host-built f32 table (:357-390,
:522-560), KV store (:446-460), scores = 0.125 * K q, softmax with max shift,
out = V^T p per q-head sharing its kv-head (lean/lib/AlgorithmLib/Cuda.lean:
313-360, Qwen2Proven.lean:666-749), Wo + residual (:988-989), rmsnorm, gate/up,
silu(g)*u (Qwen2Proven.lean:71-81), down + residual (:1019-1024), final
rmsnorm, tied lm_head, argmax = first index of the max (Qwen2Proven.lean:926-972).
Shared pieces (rms_norm, rope_rows, attention) are pinned in
tests/test_oracle_model.py against the reference's NumPy block.  The only
end-to-end golden of the reference (golden_cli.rs:17) needs the real
Qwen2-0.5B-Instruct weights, which are not available: "parity unpinned" end to
end; weights here are synthetic (oracle/synth.py).
Dot products accumulate in float64 and round once to float32 (cuBLAS, which the
reference calls for them, commits to no order: ML/Compose.lean:261-285)."""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from . import synth
from .gptoss_oracle import attn_sink, rms_norm, rope_rows, rope_table

KIND = dict(ln1=0, wqkv=1, bqkv=2, wo=3, ln2=4, wgu=5, wdn=6, embed=16, lnf=17)
GLOBAL_LAYER = 1000


@dataclass
class Cfg:
    layers: int = 24
    hidden: int = 896
    inter: int = 4864
    n_q: int = 14
    n_kv: int = 2
    vocab: int = 151936
    max_seq: int = 2048
    batch: int = 1
    rope_theta: float = 1e6
    eps: float = 1e-6
    seed: int = 0


def silu(v):
    return (v / (np.float32(1.0) + np.exp(-v))).astype(np.float32)


def make_weights(c: Cfg) -> dict:
    H, F = c.hidden, c.inter
    QD, KVD = c.n_q * 64, c.n_kv * 64
    QKV = QD + 2 * KVD
    t, s = synth.tensor_id, c.seed
    w = {"embed": synth.normal(c.vocab * H, t(GLOBAL_LAYER, 16), s, 0.02).reshape(c.vocab, H),
         "lnf": synth.one_plus_normal(H, t(GLOBAL_LAYER, 17), s, 0.02), "layers": []}
    for l in range(c.layers):
        w["layers"].append({
            "ln1": synth.one_plus_normal(H, t(l, 0), s, 0.02),
            "wqkv": synth.normal(QKV * H, t(l, 1), s, 0.02).reshape(QKV, H),
            "bqkv": synth.normal(QKV, t(l, 2), s, 0.02),
            "wo": synth.normal(H * QD, t(l, 3), s, 0.02).reshape(H, QD),
            "ln2": synth.one_plus_normal(H, t(l, 4), s, 0.02),
            "wgu": synth.normal(2 * F * H, t(l, 5), s, 0.02).reshape(2 * F, H),
            "wdn": synth.normal(H * F, t(l, 6), s, 0.02).reshape(H, F),
        })
    return w


def _mv(W, x):
    return (W.astype(np.float64) @ x.astype(np.float64)).astype(np.float32)


class Model:
    def __init__(self, c: Cfg, w: dict | None = None):
        self.c = c
        self.w = w or make_weights(c)
        self.rope = rope_table(c.rope_theta, c.max_seq)
        self.k = [np.zeros((c.n_kv, 0, 64), dtype=np.float32) for _ in range(c.layers)]
        self.v = [np.zeros((c.n_kv, 0, 64), dtype=np.float32) for _ in range(c.layers)]

    def step(self, token: int, pos: int, return_logits=False):
        c, w = self.c, self.w
        x = w["embed"][token].astype(np.float32)
        sin, cos = self.rope[0, pos], self.rope[1, pos]
        QD, KVD, F = c.n_q * 64, c.n_kv * 64, c.inter
        for l, ly in enumerate(w["layers"]):
            xn = rms_norm(ly["ln1"], x, c.eps)
            qkv = (_mv(ly["wqkv"], xn) + ly["bqkv"]).astype(np.float32)
            q = (rope_rows(qkv[:QD].reshape(c.n_q, 64), sin, cos) * np.float32(0.125)).astype(np.float32)
            kn = rope_rows(qkv[QD:QD + KVD].reshape(c.n_kv, 64), sin, cos)
            vn = qkv[QD + KVD:].reshape(c.n_kv, 64)
            self.k[l] = np.concatenate([self.k[l], kn[:, None, :]], axis=1)
            self.v[l] = np.concatenate([self.v[l], vn[:, None, :]], axis=1)
            a = attn_sink(q, self.k[l], self.v[l], None, c.n_kv).reshape(QD)
            h = (x + _mv(ly["wo"], a)).astype(np.float32)
            xn2 = rms_norm(ly["ln2"], h, c.eps)
            gu = _mv(ly["wgu"], xn2)
            act = (silu(gu[:F]) * gu[F:]).astype(np.float32)
            x = (h + _mv(ly["wdn"], act)).astype(np.float32)
        logits = _mv(w["embed"], rms_norm(w["lnf"], x, c.eps))
        nxt = int(np.argmax(logits))
        return (nxt, logits) if return_logits else nxt
