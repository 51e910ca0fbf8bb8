"""Batched decode (many sequences per GPU: dense layers and experts on the tcgen05 tensor cores, every weight
read once per step) against the oracle and against single-sequence runs, through Base/execute_into, plus the
dense skinny GEMM alone against NumPy through cl_b200_launch."""
import ctypes
import struct

import numpy as np
import pytest

from base_b200 import lib
from base_b200.gptoss import GptOss, GptOssConfig, PDL, BATCHED
from oracle import gptoss_oracle as go
from oracle import synth

pytestmark = pytest.mark.gpu
TOL_LOGITS = 1e-3


def rel(a, b):
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))


def ocfg(c: GptOssConfig):
    return go.Cfg(layers=c.layers, hidden=c.hidden, inter=c.inter, experts=c.experts, top_k=c.top_k, n_q=c.n_q,
                  n_kv=c.n_kv, vocab=c.vocab, window=c.window, max_seq=c.max_seq, batch=c.batch,
                  rope_theta=c.rope_theta, eps=c.eps, alpha=c.alpha, limit=c.limit, seed=c.seed)


def small(**kw):
    base = dict(layers=3, hidden=128, inter=192, experts=8, top_k=4, n_q=8, n_kv=2, vocab=512, window=8,
                max_seq=64, batch=1, seed=5, flags=PDL)
    base.update(kw)
    return GptOssConfig(**base)


def run_gemm(L, c, rows, K, B, kind, rows16, grid, rng):
    """out = x W^T + bias (+ res) through dense_tc_retile, rows_to_a and dense_tc_gemm."""
    mod = L.cl_b200_builtin_module(c)
    W = synth.bf16_round(rng.standard_normal((rows, K)).astype(np.float32) * 0.05)
    x = rng.standard_normal((B, K)).astype(np.float32)
    bias = rng.standard_normal(rows).astype(np.float32)
    res = rng.standard_normal((B, rows)).astype(np.float32)
    wbits = np.ascontiguousarray(synth.f32_to_bf16_bits(W.reshape(-1)))
    passes = (B + 31) // 32
    sizes = dict(w=wbits.nbytes, wt=wbits.nbytes, x=x.nbytes, at=passes * (K // 64) * 8192, bias=bias.nbytes,
                 res=res.nbytes, out=B * rows * 4, st=4)
    b = {k: L.cl_cuda_create_buffer(c, v) for k, v in sizes.items()}
    assert min(b.values()) >= 0
    for k, arr in (("w", wbits), ("x", x), ("bias", bias), ("res", res)):
        assert L.cl_cuda_upload_ptr(c, b[k], arr.ctypes.data_as(ctypes.c_void_p), arr.nbytes) == 0

    def launch(name, ids, args, gx, threads, smem=0):
        rc = L.cl_b200_launch(c, mod, name, len(ids), struct.pack(f"<{len(ids)}i", *ids), args, len(args), gx, 1, 1, threads,
                              1, 1, smem, -1, 0)
        assert rc == 0, L.cl_b200_last_error().decode()

    launch(b"dense_tc_retile", [b["w"], b["wt"]], struct.pack("<2i", rows, K), 64, 256)
    launch(b"rows_to_a", [b["x"], -1, -1, -1, -1, b["at"]], struct.pack("<4iqf4x", K, B, 0, 0, 0, 1e-5), B, 256)
    smem = 8 * (8192 + 16 * 1024) + 64 * 129 * 4 + 512
    launch(b"dense_tc_gemm", [b["wt"], b["at"], b["bias"], b["res"], b["out"], b["st"]],
           struct.pack("<6i", rows, K, B, kind, rows16, rows), grid, 192, smem)
    assert L.cl_cuda_sync(c) == 0, L.cl_b200_last_error().decode()
    st = np.zeros(1, np.int32)
    out = np.zeros((B, rows), np.float32)
    assert L.cl_cuda_download_ptr(c, b["st"], st.ctypes.data_as(ctypes.c_void_p), 4) == 0
    assert L.cl_cuda_download_ptr(c, b["out"], out.ctypes.data_as(ctypes.c_void_p), out.nbytes) == 0
    assert st[0] == 0, f"kernel gave up waiting (code {st[0]})"
    for v in b.values():
        L.cl_cuda_free_buffer(c, v)
    ref = x.astype(np.float64) @ W.astype(np.float64).T + bias + (res if kind == 1 else 0)
    return out, ref


@pytest.fixture()
def ctx():
    L = lib()
    slot = ctypes.c_void_p(0)
    L.cl_cuda_init(ctypes.byref(slot))
    assert slot.value, "no GPU? " + L.cl_b200_last_error().decode()
    yield L, slot
    L.cl_cuda_cleanup(ctypes.byref(slot))


def test_dense_gemm_accumulator_rows_and_numpy(ctx):
    """Where an M = 64 instruction puts accumulator row r (16 rows per lane quarter) is a property of the tensor
    core; the product code passes 1.  Exactly that choice must reproduce NumPy."""
    L, c = ctx
    errs = {}
    for rows16 in (1, 0):
        out, ref = run_gemm(L, c, 64, 128, 32, 0, rows16, 2, np.random.default_rng(1))   # 32 tokens: all 64 accumulator rows in use
        errs[rows16] = rel(out, ref)
    print("max-rel-err by accumulator row placement:", errs)
    assert errs[1] < 2e-5 and errs[0] > 10 * errs[1]


@pytest.mark.parametrize("rows,K,B,kind,grid", [(5120, 2880, 32, 0, 148), (2880, 4096, 7, 1, 148), (4096, 2880, 70, 0, 37),
                                                 (72, 64, 1, 1, 5), (2880, 4096, 12, 1, 148), (5120, 2880, 20, 0, 148)])
def test_dense_gemm_shapes(ctx, rows, K, B, kind, grid):
    L, c = ctx
    out, ref = run_gemm(L, c, rows, K, B, kind, 1, grid, np.random.default_rng(rows + K + B))
    assert rel(out, ref) < 2e-5


def drive_batched(c, n_steps, firsts, check_oracle=(0,), fill=False, start=0):
    """Teacher-forced on the batched instance's own tokens; sequences listed in check_oracle are compared with the
    NumPy oracle at every step."""
    m = GptOss(c)
    oracles = {b: go.Model(ocfg(c)) for b in check_oracle}
    if fill:
        m.fill_kv()
        for b, o in oracles.items():
            o.fill_kv(start, seq=b)
    toks = list(firsts)
    checked = 0
    history = []
    for pos in range(start, start + n_steps):
        got = m.infer(toks, [pos] * c.batch)
        logits = m.logits()
        for b, o in oracles.items():
            want, ref = o.step(toks[b], pos, return_logits=True)
            assert rel(logits[b], ref) < TOL_LOGITS, f"seq {b} pos {pos}: {rel(logits[b], ref)}"
            top2 = np.sort(ref)[-2:]
            if top2[1] - top2[0] > 4 * TOL_LOGITS * np.abs(ref).max():
                assert int(got[b]) == want
                checked += 1
        history.append(got.copy())
        toks = [int(t) for t in got]
    m.close()
    return np.array(history), checked


def test_batched_step_matches_oracle_small():
    c = small(batch=5, flags=PDL | BATCHED)
    _, checked = drive_batched(c, 12, [7, 99, 400, 3, 250], check_oracle=(0, 3, 4))       # the 8-row ring wraps
    assert checked > 0


def test_batched_equals_single_sequence_runs():
    firsts = [3, 99, 400, 17, 8, 301]
    cb = small(batch=len(firsts), flags=PDL | BATCHED)
    hist, _ = drive_batched(cb, 6, firsts, check_oracle=())
    for i, f in enumerate(firsts):
        s = GptOss(small())
        s.prep([f], [0])
        assert s.decode(6)[:, 0].tolist() == hist[:, i].tolist(), f"sequence {i}"
        s.close()


def test_more_tokens_than_one_pass_per_expert_and_per_gemm():
    # 40 sequences: two passes of 32 in the dense GEMMs; 160 assignments over 8 experts: more than 16 tokens per expert
    c = small(batch=40, layers=2, flags=PDL | BATCHED)
    firsts = [(37 * i + 5) % c.vocab for i in range(40)]
    _, checked = drive_batched(c, 3, firsts, check_oracle=(0, 31, 32, 39))
    assert checked > 0


def test_device_feedback_and_bounds_in_batched_mode():
    c = small(batch=4, flags=PDL | BATCHED, max_seq=16)
    a, b = GptOss(c), GptOss(c)
    toks, seq = [1, 2, 3, 4], []
    for pos in range(5):
        toks = [int(t) for t in a.infer(toks, [pos] * 4)]
        seq.append(toks)
    b.prep([1, 2, 3, 4], [0] * 4)
    assert b.decode(5).tolist() == seq
    b.prep([1, 2, 3, 4], [14] * 4)
    with pytest.raises(RuntimeError, match="out of range"):
        b.decode(3)
    a.close(), b.close()


def test_batched_full_width_against_c_oracle():
    """Two layers at the gpt-oss-20b widths, 32 sequences (benchmark config 3 at batch 32): first positions, then
    context 2047 on the synthetic KV cache, three sequences against the C oracle."""
    from oracle import c_oracle
    c = GptOssConfig(layers=2, hidden=2880, inter=2880, experts=32, top_k=4, n_q=64, n_kv=8, vocab=4096, window=128,
                     max_seq=2304, batch=32, seed=3, flags=PDL | BATCHED)
    m = GptOss(c)
    watch = (0, 13, 31)
    oracles = {b: c_oracle.GptOssC(ocfg(c)) for b in watch}
    toks = [(91 * i + 7) % c.vocab for i in range(32)]
    for pos in (0, 1):
        got = m.infer(toks, [pos] * 32)
        logits = m.logits()
        for b, o in oracles.items():
            want, ref = o.step(toks[b], pos, return_logits=True)
            assert rel(logits[b], ref) < TOL_LOGITS, f"seq {b} pos {pos}: {rel(logits[b], ref)}"
        toks = [int(t) for t in got]
    m.fill_kv()
    for b, o in oracles.items():
        o.fill_kv(seq=b, batch=32)
    for pos in (2047, 2048):
        got = m.infer(toks, [pos] * 32)
        logits = m.logits()
        for b, o in oracles.items():
            want, ref = o.step(toks[b], pos, return_logits=True)
            assert rel(logits[b], ref) < TOL_LOGITS, f"seq {b} pos {pos}: {rel(logits[b], ref)}"
            top2 = np.sort(ref)[-2:]
            if top2[1] - top2[0] > 4 * TOL_LOGITS * np.abs(ref).max():
                assert int(got[b]) == want
        toks = [int(t) for t in got]
    m.close()
    for o in oracles.values():
        o.close()


def test_few_sequences_long_context_split_over_ctas():
    # 2 sequences x 2 kv heads: the batched attention kernel gives every (sequence, kv head) several CTAs, each
    # streaming a range of slices; their partial results are merged by the last one (5 slices at position 600)
    c = small(batch=2, layers=2, max_seq=700, window=16, flags=PDL | BATCHED)
    _, checked = drive_batched(c, 3, [7, 99], check_oracle=(0, 1), fill=True, start=600)
    assert checked > 0
