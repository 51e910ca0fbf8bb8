"""CPU oracle for gpt-oss-architecture greedy decode.  TEST INFRASTRUCTURE ONLY.

What each piece restates (reference = unnamedlambda/base):
  RMSNorm    x * w * 1/sqrt(mean(x^2) + eps)   lean/algorithms/Qwen2Proven.lean:304-333,
                                               ML/Transformer.lean:101-102; NumPy image
                                               applications/ten-qwen/run.py:25-27
  RoPE       half-split pairs, host-built f32 table [sin; cos][pos][hd/2]
                                               Qwen2Proven.lean:487-511, Qwen2Common.lean:522-560,
                                               run.py:30-36
  attention  scale * K q, softmax (max shift), P^T V, q-heads share kv-heads
                                               lean/lib/AlgorithmLib/Cuda.lean:313-360, run.py:39-44
  argmax     first index of the maximum        Qwen2Proven.lean:926-972
  decode     one token per call, [token, pos]  Qwen2Common.lean:30, 830-864
`rms_norm`, `rope_rows` and `attn_plain` are checked against outputs of the
reference's own NumPy block (tests/golden/ref_block.npz).
NOT in the reference, fixed here and pinned against the gpt-oss module of the
`transformers` package (tests/golden/hf_gptoss_attn.npz): the sink logit that
enters the softmax denominator only, the sliding window (position p sees
positions > p - window), bf16 K/V storage, sliding layers first.  With respect
to the reference itself that part is "parity unpinned".
Dot products accumulate in float64 and round once to float32.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from . import moe_oracle as mo
from . import synth

KIND = dict(ln1=0, wqkv=1, bqkv=2, sinks=3, wo=4, bo=5, ln2=6, wr=7, br=8, gu_codes=9, gu_scales=10, gu_bias=11,
            dn_codes=12, dn_scales=13, dn_bias=14, embed=16, lm_head=17, lnf=18)
GLOBAL_LAYER = 1000


@dataclass
class Cfg:
    layers: int
    hidden: int
    inter: int
    experts: int
    top_k: int
    n_q: int
    n_kv: int
    vocab: int
    window: int
    max_seq: int
    batch: int = 1
    head_dim: int = 64
    rope_theta: float = 150000.0
    eps: float = 1e-5
    alpha: float = 1.702
    limit: float = 7.0
    seed: int = 0


def rms_norm(g, x, eps):
    ss = np.float32(np.sum(x.astype(np.float64) ** 2))
    inv = np.float32(1.0) / np.sqrt(ss / np.float32(x.shape[-1]) + np.float32(eps), dtype=np.float32)
    return (x * inv * g).astype(np.float32)


def rope_table(theta, max_seq, half=32):
    """[2][max_seq][half] f32: sin then cos, computed in f32 as the reference's host code does."""
    i = np.arange(half, dtype=np.float32)
    inv = np.power(np.float32(theta), -(i / np.float32(half)), dtype=np.float32)
    ang = (np.arange(max_seq, dtype=np.float32)[:, None] * inv[None, :]).astype(np.float32)
    return np.stack([np.sin(ang, dtype=np.float32), np.cos(ang, dtype=np.float32)]).astype(np.float32)


def rope_rows(x, sin, cos):
    """x [heads, hd]; sin, cos [hd/2].  lo' = lo*cos - hi*sin, hi' = lo*sin + hi*cos, f32, no fma."""
    h = x.shape[1] // 2
    lo, hi = x[:, :h], x[:, h:]
    out = np.empty_like(x)
    out[:, :h] = (lo * cos).astype(np.float32) - (hi * sin).astype(np.float32)
    out[:, h:] = (lo * sin).astype(np.float32) + (hi * cos).astype(np.float32)
    return out.astype(np.float32)


def attn_plain(kc, vc, q, scale):
    """The reference's attention (no sink): q [nq, hd] all sharing kc, vc [S, hd]."""
    sc = (q.astype(np.float64) @ kc.astype(np.float64).T * scale)
    sc = sc - sc.max(axis=1, keepdims=True)
    e = np.exp(sc)
    return ((e / e.sum(axis=1, keepdims=True)) @ vc.astype(np.float64)).astype(np.float32)


def attn_sink(q, K, V, sinks, n_kv):
    """q [NQ, hd] (already scaled); K, V [NKV, S, hd] visible positions only;
    sinks [NQ] or None.  softmax over [scores, sink], sink column dropped."""
    NQ = q.shape[0]
    G = NQ // n_kv
    out = np.zeros_like(q, dtype=np.float32)
    for qh in range(NQ):
        kv = qh // G
        sc = K[kv].astype(np.float64) @ q[qh].astype(np.float64)
        m = sc.max() if sinks is None else max(sc.max(), float(sinks[qh]))
        e = np.exp(sc - m)
        den = e.sum() + (0.0 if sinks is None else np.exp(float(sinks[qh]) - m))
        out[qh] = ((e / den) @ V[kv].astype(np.float64)).astype(np.float32)
    return out


def make_weights(c: Cfg) -> dict:
    """The tensors base_b200's `native:gptoss` load stage generates for this config."""
    H, I, E = c.hidden, c.inter, c.experts
    QD, KVD = c.n_q * 64, c.n_kv * 64
    QKV = QD + 2 * KVD
    t = synth.tensor_id
    s = c.seed
    w = {"embed": synth.normal_bf16(c.vocab * H, t(GLOBAL_LAYER, 16), s, 0.02).reshape(c.vocab, H),
         "lm_head": synth.normal_bf16(c.vocab * H, t(GLOBAL_LAYER, 17), s, 0.02).reshape(c.vocab, H),
         "lnf": synth.one_plus_normal(H, t(GLOBAL_LAYER, 18), s, 0.02), "layers": []}
    for l in range(c.layers):
        ly = {
            "ln1": synth.one_plus_normal(H, t(l, 0), s, 0.02),
            "wqkv": synth.normal_bf16(QKV * H, t(l, 1), s, 0.02).reshape(QKV, H),
            "bqkv": synth.normal(QKV, t(l, 2), s, 0.02),
            "sinks": synth.normal(c.n_q, t(l, 3), s, 1.0),
            "wo": synth.normal_bf16(H * QD, t(l, 4), s, 0.02).reshape(H, QD),
            "bo": synth.normal(H, t(l, 5), s, 0.02),
            "ln2": synth.one_plus_normal(H, t(l, 6), s, 0.02),
            "Wr": synth.normal(E * H, t(l, 7), s, 0.02).reshape(E, H),
            "br": synth.normal(E, t(l, 8), s, 0.01),
            "gu_codes": synth.bytes_(E * 2 * I * (H // 2), t(l, 9), s).reshape(E, 2 * I, H // 2),
            "gu_scales": synth.scales(E * 2 * I * (H // 32), t(l, 10), s).reshape(E, 2 * I, H // 32),
            "gu_bias": synth.normal(E * 2 * I, t(l, 11), s, 0.01).reshape(E, 2 * I),
            "dn_codes": synth.bytes_(E * H * (I // 2), t(l, 12), s).reshape(E, H, I // 2),
            "dn_scales": synth.scales(E * H * (I // 32), t(l, 13), s).reshape(E, H, I // 32),
            "dn_bias": synth.normal(E * H, t(l, 14), s, 0.01).reshape(E, H),
            "top_k": c.top_k, "alpha": c.alpha, "limit": c.limit,
            "window": c.window if l % 2 == 0 else 0,
        }
        w["layers"].append(ly)
    return w


class Model:
    """One sequence, greedy decode, token by token with a KV cache."""

    def __init__(self, c: Cfg, w: dict | None = None):
        self.c = c
        self.w = w or make_weights(c)
        self.rope = rope_table(c.rope_theta, c.max_seq)
        self.k = [np.zeros((c.n_kv, 0, 64), dtype=np.float32) for _ in range(c.layers)]
        self.v = [np.zeros((c.n_kv, 0, 64), dtype=np.float32) for _ in range(c.layers)]
        self.deq = {}

    def _expert(self, l, ly, e):
        """Dequantised (gate_up, down) matrices of expert e of layer l, a few kept."""
        if (l, e) not in self.deq:
            if len(self.deq) >= 16:
                self.deq.pop(next(iter(self.deq)))
            self.deq[(l, e)] = (mo.mx_dequant(ly["gu_codes"][e], ly["gu_scales"][e]),
                                mo.mx_dequant(ly["dn_codes"][e], ly["dn_scales"][e]))
        return self.deq[(l, e)]

    def fill_kv(self, n_pos: int, seq: int = 0):
        """The synthetic cache the stage program's `fillKV` extra writes, for positions < n_pos: every K/V row
        is bf16 N(0, 1) from (seed, layer * 32 + 19 / 20, index in [batch][n_kv][cache_len][64]); position p of a
        sliding layer sits in row p % cache_len."""
        c = self.c
        for l, ly in enumerate(self.w["layers"]):
            cache_len = min(ly["window"], c.max_seq) if ly["window"] > 0 else c.max_seq
            n = c.n_kv * cache_len * 64
            rows = np.arange(n_pos) % cache_len
            for kind, dst in ((19, self.k), (20, self.v)):
                buf = synth.normal_bf16(n * (seq + 1), synth.tensor_id(l, kind), c.seed, 1.0)[n * seq:]
                dst[l] = buf.reshape(c.n_kv, cache_len, 64)[:, rows, :].copy()

    def step(self, token: int, pos: int, return_logits=False):
        c, w = self.c, self.w
        assert all(kk.shape[1] == pos for kk in self.k), "positions must be fed in order"
        x = w["embed"][token].astype(np.float32)
        sin, cos = self.rope[0, pos], self.rope[1, pos]
        QD, KVD = c.n_q * 64, c.n_kv * 64
        for l, ly in enumerate(w["layers"]):
            xn = rms_norm(ly["ln1"], x, c.eps)
            qkv = ((ly["wqkv"].astype(np.float64) @ xn.astype(np.float64)).astype(np.float32) + ly["bqkv"]).astype(np.float32)
            q = (rope_rows(qkv[:QD].reshape(c.n_q, 64), sin, cos) * np.float32(0.125)).astype(np.float32)
            kn = synth.bf16_round(rope_rows(qkv[QD:QD + KVD].reshape(c.n_kv, 64), sin, cos))
            vn = synth.bf16_round(qkv[QD + KVD:].reshape(c.n_kv, 64))
            self.k[l] = np.concatenate([self.k[l], kn[:, None, :]], axis=1)
            self.v[l] = np.concatenate([self.v[l], vn[:, None, :]], axis=1)
            lo = max(0, pos + 1 - ly["window"]) if ly["window"] > 0 else 0
            a = attn_sink(q, self.k[l][:, lo:], self.v[l][:, lo:], ly["sinks"], c.n_kv).reshape(QD)
            h = (x + (ly["wo"].astype(np.float64) @ a.astype(np.float64)).astype(np.float32) + ly["bo"]).astype(np.float32)
            xn2 = rms_norm(ly["ln2"], h, c.eps)
            logits = mo.router_logits(xn2[None, :], ly["Wr"], ly["br"])
            idx, wt = mo.topk_softmax(logits, c.top_k)
            y = np.zeros(c.hidden, dtype=np.float32)
            for j in range(c.top_k):
                e = int(idx[0, j])
                guw, dnw = self._expert(l, ly, e)
                o, _ = mo.expert_ffn(xn2, guw, ly["gu_bias"][e], dnw, ly["dn_bias"][e], c.alpha, c.limit)
                y = (y + wt[0, j] * o).astype(np.float32)
            x = (h + y).astype(np.float32)
        xf = rms_norm(w["lnf"], x, c.eps)
        logits = (w["lm_head"].astype(np.float64) @ xf.astype(np.float64)).astype(np.float32)
        nxt = int(np.argmax(logits))          # numpy returns the first index of the maximum
        return (nxt, logits) if return_logits else nxt
