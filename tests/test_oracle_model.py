"""Model-level oracle pieces vs the reference's own NumPy block and the
transformers gpt-oss attention fixture (CPU)."""
import numpy as np

from oracle import gptoss_oracle as go
from oracle import synth


def _ref_block_weights(seed=7):
    # the recipe of applications/ten-qwen/run.py:66-83 (make_weights)
    DM, NH, HD, SQ, DFF = 512, 8, 64, 128, 1408
    r = np.random.default_rng(seed)

    def u(*shape):
        return (r.standard_normal(shape) * 0.02).astype(np.float32)
    ang = (np.arange(HD // 2, dtype=np.float32) + 1.0) * 0.11
    w = {"cos": np.cos(ang).astype(np.float32), "sin": np.sin(ang).astype(np.float32)}
    w["ones"] = np.ones(SQ, dtype=np.float32)
    w["kc"], w["vc"], w["x"] = u(SQ, HD), u(SQ, HD), u(DM)
    w["g1"] = (1.0 + u(DM)).astype(np.float32)
    w["g2"] = (1.0 + u(DM)).astype(np.float32)
    w["wq"], w["wo"] = u(DM, DM), u(DM, DM)
    return w, (DM, NH, HD, SQ, DFF)


def test_rmsnorm_rope_attention_vs_reference_block(golden):
    g = np.load(golden / "ref_block.npz")
    w, (DM, NH, HD, SQ, DFF) = _ref_block_weights()
    assert [int(v) for v in g["dims"]] == [DM, NH, HD, SQ, DFF]
    n1 = go.rms_norm(w["g1"], w["x"], 1e-6)                          # run.py:25-27 uses eps 1e-6
    np.testing.assert_allclose(n1, g["n1"], rtol=2e-6, atol=1e-7)
    q = go.rope_rows((w["wq"] @ g["n1"]).astype(np.float32).reshape(NH, HD), w["sin"], w["cos"])
    np.testing.assert_allclose(q, g["q"], rtol=1e-5, atol=1e-7)
    a = go.attn_plain(w["kc"], w["vc"], g["q"], 1.0 / np.sqrt(HD))
    np.testing.assert_allclose(a, g["attn"], rtol=2e-5, atol=1e-7)


def test_sink_attention_vs_transformers_fixture(golden):
    g = np.load(golden / "hf_gptoss_attn.npz")
    NQ, NKV, HD, S = [int(v) for v in g["dims"]]
    r = np.random.default_rng(303)
    q = r.standard_normal((1, NQ, 1, HD)).astype(np.float32)
    k = r.standard_normal((1, NKV, S, HD)).astype(np.float32)
    v = r.standard_normal((1, NKV, S, HD)).astype(np.float32)
    sinks = r.standard_normal(NQ).astype(np.float32)
    qs = (q[0, :, 0, :] * np.float32(HD ** -0.5)).astype(np.float32)
    full = go.attn_sink(qs, k[0], v[0], sinks, NKV)
    np.testing.assert_allclose(full, g["full"], rtol=2e-5, atol=2e-6)
    win = go.attn_sink(qs, k[0][:, S - 16:], v[0][:, S - 16:], sinks, NKV)
    np.testing.assert_allclose(win, g["win16"], rtol=2e-5, atol=2e-6)
    # the sink must matter, otherwise the fixture pins nothing
    assert np.abs(go.attn_sink(qs, k[0], v[0], None, NKV) - g["full"]).max() > 1e-3


def test_synth_generator_properties():
    b = synth.bytes_(1 << 16, 5, 1)
    assert b.dtype == np.uint8 and abs(b.mean() - 127.5) < 2 and len(np.unique(b)) == 256
    s = synth.scales(10000, 6, 1)
    assert s.min() == 117 and s.max() == 123
    z = synth.normal(1 << 16, 7, 1, 0.02)
    assert abs(z.mean()) < 5e-4 and abs(z.std() / 0.02 - 1) < 0.02
    assert not np.array_equal(synth.normal(64, 7, 1, 0.02), synth.normal(64, 7, 2, 0.02))
    # round to nearest even on the 16 dropped bits: 1 + 2^-8 is a tie and goes down to 1,
    # 1 + 3 * 2^-8 is a tie and goes up to 1 + 2^-6
    x = np.array([1.0, 1.00390625, 1.01171875, -2.5], dtype=np.float32)
    assert synth.bf16_round(x).tolist() == [1.0, 1.0, 1.015625, -2.5]
    big = synth.bf16_round(np.array([3.0e38], dtype=np.float32))
    assert np.isfinite(big).all() and abs(float(big[0]) / 3.0e38 - 1) < 2 ** -8


def test_tiny_model_runs_and_is_deterministic():
    c = go.Cfg(layers=2, hidden=64, inter=64, experts=4, top_k=2, n_q=2, n_kv=1, vocab=50, window=4, max_seq=16)
    m1, m2 = go.Model(c), go.Model(c)
    t1 = [m1.step(3 + i, i) for i in range(6)]
    t2 = [m2.step(3 + i, i) for i in range(6)]
    assert t1 == t2 and all(0 <= t < 50 for t in t1)


# ---- the C restatement of whole decode steps (oracle/model_oracle.c) against the NumPy oracles ----
def _rel(a, b):
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))


def test_c_gptoss_model_matches_numpy_model():
    from oracle import c_oracle
    c = go.Cfg(layers=3, hidden=128, inter=192, experts=8, top_k=4, n_q=8, n_kv=2, vocab=300, window=8, max_seq=40, seed=5)
    a, b = go.Model(c), c_oracle.GptOssC(c, threads=2)
    tok = 7
    for pos in range(20):                                   # the sliding layers' ring (8 rows) wraps twice
        ta, la = a.step(tok, pos, return_logits=True)
        tb, lb = b.step(tok, pos, return_logits=True)
        assert _rel(lb, la) < 2e-5, f"pos {pos}"
        top2 = np.sort(la)[-2:]
        if top2[1] - top2[0] > 1e-4 * np.abs(la).max():
            assert ta == tb
        tok = ta
    st = b.stats()
    assert st["experts"].shape == (3, 4) and st["moe_s"] > 0
    b.close()


def test_c_gptoss_synthetic_cache_matches_numpy_fill():
    from oracle import c_oracle
    c = go.Cfg(layers=2, hidden=128, inter=64, experts=4, top_k=2, n_q=4, n_kv=2, vocab=100, window=16, max_seq=300, seed=9)
    a, b = go.Model(c), c_oracle.GptOssC(c, threads=2)
    a.fill_kv(270)
    b.fill_kv()
    for pos, tok in ((270, 3), (271, 50)):
        _, la = a.step(tok, pos, return_logits=True)
        _, lb = b.step(tok, pos, return_logits=True)
        assert _rel(lb, la) < 2e-5
    # the filled rows matter: an empty cache gives different logits at the same position
    e = go.Model(c)
    e.k = [np.zeros((c.n_kv, 270, 64), dtype=np.float32) for _ in range(c.layers)]
    e.v = [np.zeros((c.n_kv, 270, 64), dtype=np.float32) for _ in range(c.layers)]
    _, le = e.step(3, 270, return_logits=True)
    a2 = go.Model(c)
    a2.fill_kv(270)
    _, la2 = a2.step(3, 270, return_logits=True)
    assert _rel(le, la2) > 1e-3
    b.close()


def test_c_qwen2_model_matches_numpy_model():
    from oracle import c_oracle
    from oracle import qwen2_oracle as qo
    c = qo.Cfg(layers=2, hidden=128, inter=256, n_q=4, n_kv=2, vocab=400, max_seq=24, seed=3)
    a, b = qo.Model(c), c_oracle.Qwen2C(c, threads=2)
    tok = 11
    for pos in range(12):
        ta, la = a.step(tok, pos, return_logits=True)
        tb, lb = b.step(tok, pos, return_logits=True)
        assert _rel(lb, la) < 2e-5, f"pos {pos}"
        top2 = np.sort(la)[-2:]
        if top2[1] - top2[0] > 1e-4 * np.abs(la).max():
            assert ta == tb
        tok = ta
    b.close()


def test_rowdot_fold_is_the_reference_cpu_gemv_order():
    # lean/algorithms/RowDotBenchAlgorithm.lean:86-121: four lane accumulators acc_j += x * w (separate
    # multiply and add), (e0 + e1) + (e2 + e3), then a scalar tail; restated here in NumPy f32
    from oracle import c_oracle
    r = np.random.default_rng(4)
    for K in (896, 2880, 2883):
        W = r.standard_normal((5, K)).astype(np.float32)
        x = r.standard_normal(K).astype(np.float32)
        want = np.zeros(5, dtype=np.float32)
        for i in range(5):
            acc = np.zeros(4, dtype=np.float32)
            n4 = K // 4 * 4
            for j in range(0, n4, 4):
                acc = (acc + (x[j:j + 4] * W[i, j:j + 4]).astype(np.float32)).astype(np.float32)
            s = np.float32(np.float32(acc[0] + acc[1]) + np.float32(acc[2] + acc[3]))
            for j in range(n4, K):
                s = np.float32(s + np.float32(x[j] * W[i, j]))
            want[i] = s
        got = c_oracle.rowdot_gemv(W, x, threads=1)
        np.testing.assert_array_equal(got.view(np.uint32), want.view(np.uint32))
        np.testing.assert_array_equal(c_oracle.rowdot_gemv(W, x, threads=3).view(np.uint32), want.view(np.uint32))


def test_warp_fold_restatement_matches_the_reference_unit_tests():
    # applications/warp-check/src/lib.rs:260-281: the three walks cover the same indices (the folds agree on
    # exactly representable data) and the butterfly sums 32 ones to 32
    from oracle import c_oracle
    ones = np.ones((1, 256), dtype=np.float32)
    for walk in (0, 1, 2):
        assert c_oracle.warp_fold_gemv(ones, ones[0], walk)[0] == 256.0
    a = (np.arange(3 * 1024) % 7).astype(np.float32).reshape(3, 1024)
    x = (np.arange(1024) % 5).astype(np.float32)
    want = (a.astype(np.float64) @ x.astype(np.float64)).astype(np.float32)
    for walk in (0, 1, 2):
        np.testing.assert_array_equal(c_oracle.warp_fold_gemv(a, x, walk), want)     # small integers: every order is exact
    # and on data that is not exactly summable the walks differ in the last bits, as the reference says they do
    r = np.random.default_rng(0)
    b, z = r.standard_normal((4, 4096)).astype(np.float32), r.standard_normal(4096).astype(np.float32)
    assert not np.array_equal(c_oracle.warp_fold_gemv(b, z, 0), c_oracle.warp_fold_gemv(b, z, 1))
