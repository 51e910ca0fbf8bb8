"""ctypes binding of oracle/_build/liboracle.so (the C restatement).  Test
infrastructure only."""
from __future__ import annotations

import ctypes
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
LIB = HERE / "_build" / "liboracle.so"
_lib = None


def build() -> Path:
    srcs = list(HERE.glob("*.c"))
    if not LIB.exists() or any(s.stat().st_mtime > LIB.stat().st_mtime for s in srcs):
        subprocess.run(["make", "-C", str(HERE), "-s"], check=True)
    return LIB


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(str(LIB))
        _lib.oracle_moe_ffn.restype = ctypes.c_int
        _lib.oracle_max_threads.restype = ctypes.c_int
        _lib.oracle_gptoss_new.restype = ctypes.c_void_p
        _lib.oracle_qwen2_new.restype = ctypes.c_void_p
        _lib.oracle_gptoss_step.restype = ctypes.c_int
        _lib.oracle_qwen2_step.restype = ctypes.c_int
    return _lib


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def moe_ffn(x: np.ndarray, p: dict, threads: int = 0):
    """Same contract as oracle.moe_oracle.moe_ffn; returns (y, idx, w)."""
    L = lib()
    x = np.ascontiguousarray(x, dtype=np.float32)
    T, H = x.shape
    E = p["Wr"].shape[0]
    I = p["dn_codes"].shape[2] * 2
    k = int(p["top_k"])
    arrs = {n: np.ascontiguousarray(p[n]) for n in
            ("Wr", "br", "gu_codes", "gu_scales", "gu_bias", "dn_codes", "dn_scales", "dn_bias")}
    y = np.zeros((T, H), dtype=np.float32)
    idx = np.zeros((T, k), dtype=np.int32)
    w = np.zeros((T, k), dtype=np.float32)
    rc = L.oracle_moe_ffn(_p(x), T, H, I, E, k, ctypes.c_float(p.get("alpha", 1.702)),
                          ctypes.c_float(p.get("limit", 7.0)), _p(arrs["Wr"]), _p(arrs["br"]),
                          _p(arrs["gu_codes"]), _p(arrs["gu_scales"]), _p(arrs["gu_bias"]),
                          _p(arrs["dn_codes"]), _p(arrs["dn_scales"]), _p(arrs["dn_bias"]),
                          _p(y), _p(idx), _p(w), threads)
    if rc != 0:
        raise RuntimeError("oracle_moe_ffn failed")
    return y, idx, w


def max_threads() -> int:
    return lib().oracle_max_threads()


class GptOssC:
    """oracle/model_oracle.c: one sequence of a gpt-oss-architecture model with the seeded synthetic
    weights, greedy decode token by token (same contract as oracle.gptoss_oracle.Model)."""

    def __init__(self, c, threads: int = 0):
        L = lib()
        ci = (ctypes.c_int32 * 10)(c.layers, c.hidden, c.inter, c.experts, c.top_k, c.n_q, c.n_kv, c.vocab, c.window, c.max_seq)
        cf = (ctypes.c_float * 4)(c.rope_theta, c.eps, c.alpha, c.limit)
        self.c, self.L, self.threads = c, L, threads
        self.h = L.oracle_gptoss_new(ci, cf, ctypes.c_uint32(c.seed), threads)
        if not self.h:
            raise MemoryError("oracle_gptoss_new failed")

    def fill_kv(self, seq: int = 0, batch: int = 1):
        self.L.oracle_gptoss_fill_kv(ctypes.c_void_p(self.h), seq, batch)

    def step(self, token: int, pos: int, return_logits=False):
        logits = np.empty(self.c.vocab, dtype=np.float32) if return_logits else None
        nxt = self.L.oracle_gptoss_step(ctypes.c_void_p(self.h), int(token), int(pos), _p(logits) if return_logits else None, self.threads)
        if nxt < 0:
            raise RuntimeError("oracle_gptoss_step failed")
        return (nxt, logits) if return_logits else nxt

    def stats(self) -> dict:
        out = np.zeros(4 + 8 * self.c.layers, dtype=np.float64)
        self.L.oracle_gptoss_stats(ctypes.c_void_p(self.h), _p(out))
        return {"dense_s": out[0], "attention_s": out[1], "moe_s": out[2], "head_s": out[3],
                "experts": out[4:].astype(np.int64).reshape(self.c.layers, 8)[:, :self.c.top_k]}

    def close(self):
        if self.h:
            self.L.oracle_gptoss_free(ctypes.c_void_p(self.h))
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Qwen2C:
    """oracle/model_oracle.c: Qwen2-architecture greedy decode (f32), as oracle.qwen2_oracle.Model."""

    def __init__(self, c, threads: int = 0):
        L = lib()
        ci = (ctypes.c_int32 * 7)(c.layers, c.hidden, c.inter, c.n_q, c.n_kv, c.vocab, c.max_seq)
        cf = (ctypes.c_float * 2)(c.rope_theta, c.eps)
        self.c, self.L, self.threads = c, L, threads
        self.h = L.oracle_qwen2_new(ci, cf, ctypes.c_uint32(c.seed), threads)
        if not self.h:
            raise MemoryError("oracle_qwen2_new failed")

    def step(self, token: int, pos: int, return_logits=False):
        logits = np.empty(self.c.vocab, dtype=np.float32) if return_logits else None
        nxt = self.L.oracle_qwen2_step(ctypes.c_void_p(self.h), int(token), int(pos), _p(logits) if return_logits else None, self.threads)
        if nxt < 0:
            raise RuntimeError("oracle_qwen2_step failed")
        return (nxt, logits) if return_logits else nxt

    def close(self):
        if self.h:
            self.L.oracle_qwen2_free(ctypes.c_void_p(self.h))
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def rowdot_gemv(W: np.ndarray, x: np.ndarray, threads: int = 1) -> np.ndarray:
    """The reference's CPU GEMV fold (RowDotBenchAlgorithm.lean:20-150) over W [rows][K] f32."""
    W = np.ascontiguousarray(W, dtype=np.float32)
    x = np.ascontiguousarray(x, dtype=np.float32)
    y = np.empty(W.shape[0], dtype=np.float32)
    lib().oracle_rowdot_gemv_f32(_p(W), _p(x), _p(y), W.shape[0], W.shape[1], threads)
    return y


def warp_fold_gemv(W: np.ndarray, x: np.ndarray, walk: int) -> np.ndarray:
    """The reference's committed warp fold (applications/warp-check/src/lib.rs:28-116) over W [rows][n] f32."""
    W = np.ascontiguousarray(W, dtype=np.float32)
    x = np.ascontiguousarray(x, dtype=np.float32)
    y = np.empty(W.shape[0], dtype=np.float32)
    lib().oracle_warp_fold_gemv(_p(W), _p(x), _p(y), W.shape[0], W.shape[1], walk)
    return y
