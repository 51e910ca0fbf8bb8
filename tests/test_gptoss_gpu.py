"""gpt-oss decode through Base/execute_into vs the oracle.  Bit-exact: the
synthetic tensors, the dequantised expert rows, greedy tokens wherever the
oracle's top-2 logit margin exceeds the error bound.  Tolerance: logits
max|d|/max|ref| <= 1e-3 (bf16 weights and KV, f32 accumulation, f32 activations)."""
import struct

import numpy as np
import pytest

from base_b200.gptoss import GptOss, GptOssConfig, PDL, PERSISTENT, BLOCK_SCALED
from oracle import gptoss_oracle as go
from oracle import moe_oracle as mo
from oracle import synth

pytestmark = pytest.mark.gpu

TOL_LOGITS = 1e-3

# The implementations of the step: one launch per operation, the single persistent
# kernel (batch 1 only), and the persistent kernel with the experts on the block-scaled
# tensor cores.
STEP_FLAGS = [pytest.param(PDL, id="per-op"), pytest.param(PDL | PERSISTENT, id="persistent"),
              pytest.param(PDL | PERSISTENT | BLOCK_SCALED, id="persistent-block-scaled")]


def small(**kw):
    base = dict(layers=4, hidden=128, inter=192, experts=8, top_k=4, n_q=8, n_kv=2, vocab=512, window=8,
                max_seq=64, batch=1, seed=5, flags=PDL)
    base.update(kw)
    return GptOssConfig(**base)


def ocfg(c: GptOssConfig):
    return go.Cfg(layers=c.layers, hidden=c.hidden, inter=c.inter, experts=c.experts, top_k=c.top_k, n_q=c.n_q,
                  n_kv=c.n_kv, vocab=c.vocab, window=c.window, max_seq=c.max_seq, batch=c.batch,
                  rope_theta=c.rope_theta, eps=c.eps, alpha=c.alpha, limit=c.limit, seed=c.seed)


def rel(a, b):
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))


def test_synthetic_tensors_and_dequant_are_bit_exact():
    c = small()
    m = GptOss(c)
    w = go.make_weights(ocfg(c))
    H, QKV = c.hidden, (c.n_q + 2 * c.n_kv) * 64
    got = m.tensor(1000, "embed", c.vocab * H * 2, "<u2")
    np.testing.assert_array_equal(got, synth.f32_to_bf16_bits(w["embed"].reshape(-1)))
    got = m.tensor(2, "wqkv", QKV * H * 2, "<u2")
    np.testing.assert_array_equal(got, synth.f32_to_bf16_bits(w["layers"][2]["wqkv"].reshape(-1)))
    for name, key in (("ln1", "ln1"), ("bqkv", "bqkv"), ("sinks", "sinks"), ("wr", "Wr"), ("gu_bias", "gu_bias")):
        ref = w["layers"][1][key].reshape(-1)
        got = m.tensor(1, name, ref.size * 4, "<f4")
        np.testing.assert_array_equal(got.view(np.uint32), ref.view(np.uint32), err_msg=name)
    for which, ck, sk in ((0, "gu_codes", "gu_scales"), (1, "dn_codes", "dn_scales")):
        ly = w["layers"][3]
        got = m.dequant(3, which, 5, 16, 48)
        want = mo.mx_dequant(ly[ck][5, 16:64], ly[sk][5, 16:64])
        np.testing.assert_array_equal(got.view(np.uint32), want.view(np.uint32))
    m.close()


def drive(c, n_steps, first_token=7):
    """Teacher-forced: the oracle's token is fed at every step."""
    m = GptOss(c)
    o = go.Model(ocfg(c))
    tok, checked = first_token, 0
    for pos in range(n_steps):
        want, ref_logits = o.step(tok, pos, return_logits=True)
        got = int(m.infer([tok], [pos])[0])
        logits = m.logits()[0]
        assert rel(logits, ref_logits) < TOL_LOGITS, f"pos {pos}"
        top2 = np.sort(ref_logits)[-2:]
        if top2[1] - top2[0] > 4 * TOL_LOGITS * np.abs(ref_logits).max():
            assert got == want, f"pos {pos}"
            checked += 1
        else:
            assert got == int(np.argmax(logits))
        tok = want
    m.close()
    return checked


@pytest.mark.parametrize("flags", STEP_FLAGS)
def test_teacher_forced_decode_matches_oracle(flags):
    # window 8 < 24 steps: the sliding layers' ring cache wraps three times
    assert drive(small(flags=flags), 24) > 0


@pytest.mark.parametrize("flags", STEP_FLAGS)
def test_split_kv_beyond_one_slice(flags):
    # positions past 256 use two KV slices merged by the last CTA
    c = small(layers=2, max_seq=320, window=16, flags=flags)
    m = GptOss(c)
    o = go.Model(ocfg(c))
    rng = np.random.default_rng(3)
    toks = rng.integers(0, c.vocab, size=300)
    for pos in range(300):
        want, ref_logits = o.step(int(toks[pos]), pos, return_logits=True)
        m.infer([int(toks[pos])], [pos])
        if pos in (0, 255, 256, 257, 299):
            assert rel(m.logits()[0], ref_logits) < TOL_LOGITS, f"pos {pos}"
    m.close()


@pytest.mark.parametrize("flags", STEP_FLAGS)
def test_device_side_feedback_equals_step_by_step(flags):
    c = small(flags=flags)
    a, b = GptOss(c), GptOss(c)
    tok, seq = 11, []
    for pos in range(12):
        tok = int(a.infer([tok], [pos])[0])
        seq.append(tok)
    b.prep([11], [0])
    got = b.decode(12)[:, 0].tolist()
    assert got == seq
    a.close(), b.close()


def test_batch_of_sequences_is_independent():
    c1, c3 = small(), small(batch=3)
    single = GptOss(c1)
    multi = GptOss(c3)
    firsts = [3, 99, 400]
    want = []
    for f in firsts:
        s = GptOss(c1)
        s.prep([f], [0])
        want.append(s.decode(6)[:, 0].tolist())
        s.close()
    multi.prep(firsts, [0, 0, 0])
    got = multi.decode(6)
    for i in range(3):
        assert got[:, i].tolist() == want[i]
    single.close(), multi.close()


def test_persistent_step_matches_per_op_step_at_full_width():
    # two layers at the gpt-oss-20b widths (45-chunk MXFP4 tiles, 64 q heads, a
    # 4096-wide o-proj input), more than one KV slice: same tokens, same logits
    base = dict(layers=2, hidden=2880, inter=2880, experts=32, top_k=4, n_q=64, n_kv=8, vocab=4096, window=128,
                max_seq=512, batch=1, seed=3)
    a, b = GptOss(GptOssConfig(**base, flags=PDL)), GptOss(GptOssConfig(**base, flags=PDL | PERSISTENT))
    tok = 7
    for pos in list(range(4)) + [300, 301]:
        ta, tb = int(a.infer([tok], [pos])[0]), int(b.infer([tok], [pos])[0])
        assert rel(b.logits()[0], a.logits()[0]) < 1e-4, f"pos {pos}"
        assert ta == tb
        tok = ta
    times = b.phase_times(b.trace_ctas())
    assert times["layer_us"] > 0 and times["gate_up"] > 0
    a.close(), b.close()


FULL_WIDTH = dict(layers=2, hidden=2880, inter=2880, experts=32, top_k=4, n_q=64, n_kv=8, vocab=4096, window=128,
                  max_seq=2304, batch=1, seed=3)


@pytest.mark.parametrize("flags", STEP_FLAGS)
def test_full_width_steps_match_oracle_up_to_context_2048(flags):
    """Two layers at the gpt-oss-20b widths (45-chunk MXFP4 rows, 152/160-row block-scaled instructions, 64 q / 8
    kv heads, a 4096-wide o-proj input) against the C oracle: the first positions, then, on a synthetic KV cache
    that both sides generate from the seed, positions around the first KV-slice boundaries and around 2048
    (17 slices merged, the sliding layers' ring wrapped 16 times)."""
    from oracle import c_oracle
    c = GptOssConfig(**FULL_WIDTH, flags=flags)
    m, o = GptOss(c), c_oracle.GptOssC(ocfg(c))
    checked = 0

    def step(tok, pos):
        nonlocal checked
        want, ref = o.step(tok, pos, return_logits=True)
        got = int(m.infer([tok], [pos])[0])
        logits = m.logits()[0]
        assert rel(logits, ref) < TOL_LOGITS, f"pos {pos}: {rel(logits, ref)}"
        top2 = np.sort(ref)[-2:]
        if top2[1] - top2[0] > 4 * TOL_LOGITS * np.abs(ref).max():
            assert got == want, f"pos {pos}"
            checked += 1
        return want

    tok = 7
    for pos in range(4):
        tok = step(tok, pos)
    m.fill_kv()
    o.fill_kv()
    for pos in (127, 128, 129, 255, 256, 257, 2046, 2047, 2048, 2049, 2200):
        tok = step(tok, pos)
    assert checked > 0
    m.close(), o.close()


@pytest.mark.parametrize("flags", STEP_FLAGS)
def test_128_free_running_greedy_steps_match_oracle(flags):
    """128 greedy steps with the argmax fed back on the device.  The oracle is fed the device's tokens and must
    choose the same next token at every step whose top-2 margin exceeds twice the logit error bound; a second
    instance replays the sequence step by step so that the bound itself is checked at every step."""
    from oracle import c_oracle
    GUARD = 1e-4
    c = small(max_seq=160, flags=flags)
    a, b, o = GptOss(c), GptOss(c), c_oracle.GptOssC(ocfg(c))
    first = 11
    a.prep([first], [0])
    seq = a.decode(128)[:, 0].tolist()
    tok, guarded, margins = first, 0, []
    for pos in range(128):
        want, ref = o.step(tok, pos, return_logits=True)
        assert int(b.infer([tok], [pos])[0]) == seq[pos]
        scale = float(np.abs(ref).max())
        assert rel(b.logits()[0], ref) < GUARD, f"pos {pos}"
        top2 = np.sort(ref)[-2:]
        margins.append(float(top2[1] - top2[0]) / scale)
        if margins[-1] > 2 * GUARD:
            assert seq[pos] == want, f"pos {pos}: margin {margins[-1]:.2e}"
            guarded += 1
        tok = seq[pos]
    print(f"top-2 margins / max|logit|: min {min(margins):.2e}, median {np.median(margins):.2e}; {guarded}/128 steps decided")
    assert guarded >= 120
    a.close(), b.close(), o.close()


def test_steps_past_the_end_of_the_cache_are_refused():
    c = small(max_seq=16)
    m = GptOss(c)
    m.prep([1], [13])
    assert m.decode(2).shape == (2, 1)              # positions 13 and 14
    assert m.decode(1).shape == (1, 1)              # position 15, the last one
    with pytest.raises(RuntimeError, match="out of range"):
        m.decode(1)
    m.prep([1], [14])
    with pytest.raises(RuntimeError, match="out of range"):
        m.decode(3)
    m.infer([1], [15])
    with pytest.raises(RuntimeError, match="out of range"):
        m.base.execute_into(m.art.extras["infer"], b"", bytearray(4))
    m.close()


def test_load_can_be_repeated_and_a_failed_load_leaves_no_memory_behind(monkeypatch):
    import ctypes
    from base_b200 import lib
    L = lib()
    probe = ctypes.c_void_p(0)
    L.cl_cuda_init(ctypes.byref(probe))
    c = small(layers=4)
    m = GptOss(c)
    t1 = int(m.infer([5], [0])[0])
    m.base.execute(m.art.main, c.header())          # load again on a loaded instance
    assert int(m.infer([5], [0])[0]) == t1
    m.close()
    free0 = L.cl_b200_mem_free(probe)
    b = GptOss.__new__(GptOss)
    from base_b200 import py_base
    b.cfg, b.art = c, py_base.native_artifact("gptoss")
    b.base = py_base.Base(b.art.setup)
    monkeypatch.setenv("B200_TEST_FAIL_LOAD", "3")   # fails after three of the four layers are on the device
    with pytest.raises(RuntimeError, match="failure requested"):
        b.base.execute(b.art.main, c.header())
    assert L.cl_b200_mem_free(probe) >= free0 - (1 << 20)
    monkeypatch.delenv("B200_TEST_FAIL_LOAD")
    b.base.execute(b.art.main, c.header())          # the same instance loads after the failure
    assert int(b.infer([5], [0])[0]) == t1
    b.close()
    L.cl_cuda_cleanup(ctypes.byref(probe))


@pytest.mark.parametrize("flags", STEP_FLAGS[1:])
def test_a_wait_that_runs_out_is_reported_and_the_device_stays_usable(flags):
    """The persistent kernel's producers leave out one ring fill (a test hook in the load header), so the
    consumers' bounded wait for it gives up: the kernel stores a status code and ends, `infer` raises, and a
    fresh instance on the same device decodes normally afterwards."""
    c = small(layers=2, flags=flags, test_skip_fill=3, test_spin=20000)
    m = GptOss(c)
    with pytest.raises(RuntimeError, match="gave up waiting"):
        m.infer([7], [0])
    m.close()
    ok = GptOss(small(layers=2, flags=flags))
    ref = GptOss(small(layers=2, flags=PDL))
    assert int(ok.infer([7], [0])[0]) == int(ref.infer([7], [0])[0])
    ok.close(), ref.close()


def test_persistent_step_needs_batch_one():
    with pytest.raises(RuntimeError, match="batch must be 1"):
        GptOss(small(batch=2, flags=PDL | PERSISTENT))


def test_bad_requests_are_reported():
    c = small()
    m = GptOss(c)
    with pytest.raises(RuntimeError, match="out of range"):
        m.infer([c.vocab], [0])
    with pytest.raises(RuntimeError, match="out of range"):
        m.infer([1], [c.max_seq])
    m.close()


@pytest.mark.parametrize("flags", STEP_FLAGS)
def test_capture_replay_and_the_launch_ladder(flags):
    """The reference's graph extras (lean/algorithms/MlpCifarAlgorithm.lean:2233-2264) and its launch-ladder profile
    (applications/ten-qwen/profile.py:67-90): a replayed graph gives bit-identical logits to the launched step, and the
    cumulative time of the launch prefixes does not decrease."""
    c = small(flags=flags)
    a, b = GptOss(c), GptOss(c)
    n = a.capture()
    assert n == (1 if flags & PERSISTENT else 1 + c.layers * 6 + 2)
    a.infer([7], [0])
    ref = a.logits()[0].copy()
    b.prep([7], [0])
    assert b.replay(1) > 0
    np.testing.assert_array_equal(b.logits()[0].view(np.uint32), ref.view(np.uint32))
    b.prep([7], [0])
    b.run_to(n)                                      # the same launches without the graph
    np.testing.assert_array_equal(b.logits()[0].view(np.uint32), ref.view(np.uint32))
    rungs = sorted({1, max(1, n // 2), n})
    b.prep([7], [0])
    rows = b.launch_ladder(rungs, reps=5)
    assert [r[1] for r in rows] == rungs and all(r[2] > 0 for r in rows)
    assert rows[-1][2] >= rows[0][2] * 0.8
    a.close(), b.close()


@pytest.mark.parametrize("flags", [pytest.param(PDL, id="per-op"), pytest.param(PDL | PERSISTENT | BLOCK_SCALED, id="persistent-block-scaled"),
                                   pytest.param(PDL | 128, id="batched")])
def test_weights_from_a_file_replace_the_seeded_ones(flags, tmp_path):
    """base_b200/convert.py end to end: random tensors, experts quantised to MXFP4 by the converter, written as the flat
    weight file, streamed into a loaded instance with `setTensor`, decoded, and compared with the oracle run on the
    very same tensors."""
    from base_b200 import convert as cv
    from test_convert_cpu import random_weights
    c = small(layers=2, flags=flags, batch=2 if flags & 128 else 1)
    w = random_weights(c, seed=11)
    path = tmp_path / "weights.bin"
    cv.write_checkpoint(path, c, w)
    m = GptOss(c)
    before = m.infer([7] * c.batch, [0] * c.batch)
    cv.load_checkpoint(m, path)
    o = go.Model(ocfg(c), w=w)
    tok = 7
    for pos in range(6):
        want, ref = o.step(tok, pos, return_logits=True)
        got = m.infer([tok] * c.batch, [pos] * c.batch)
        assert rel(m.logits()[0], ref) < TOL_LOGITS, f"pos {pos}"
        top2 = np.sort(ref)[-2:]
        if top2[1] - top2[0] > 4 * TOL_LOGITS * np.abs(ref).max():
            assert int(got[0]) == want
        tok = want
    assert before is not None
    with pytest.raises(RuntimeError, match="expected"):
        m.base.execute(m.art.extras["setTensor"], struct.pack("<2I", 0, 0) + b"\0" * 12)
    m.close()
