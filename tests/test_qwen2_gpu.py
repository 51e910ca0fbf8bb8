"""Qwen2-architecture f32 decode through Base/execute_into vs the oracle
(benchmark config 1 shapes scaled down, plus one step at the real shapes).
Tolerance: logits max|d|/max|ref| <= 1e-4 (f32); greedy tokens identical
wherever the oracle's top-2 margin exceeds the bound."""
import numpy as np
import pytest

from base_b200.qwen2 import Qwen2, Qwen2Config
from oracle import qwen2_oracle as qo

pytestmark = pytest.mark.gpu
TOL = 1e-4


def ocfg(c):
    return qo.Cfg(layers=c.layers, hidden=c.hidden, inter=c.inter, n_q=c.n_q, n_kv=c.n_kv, vocab=c.vocab,
                  max_seq=c.max_seq, batch=c.batch, rope_theta=c.rope_theta, eps=c.eps, seed=c.seed)


def rel(a, b):
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))


def small(**kw):
    base = dict(layers=3, hidden=128, inter=320, n_q=14, n_kv=2, vocab=1000, max_seq=200, seed=3)
    base.update(kw)
    return Qwen2Config(**base)


def test_weights_are_the_oracles_bit_for_bit():
    c = small()
    m = Qwen2(c)
    w = qo.make_weights(ocfg(c))
    for name, ref in (("wqkv", w["layers"][1]["wqkv"]), ("wdn", w["layers"][2]["wdn"]), ("ln2", w["layers"][0]["ln2"])):
        lay = {"wqkv": 1, "wdn": 2, "ln2": 0}[name]
        got = m.tensor(lay, name, ref.size)
        np.testing.assert_array_equal(got.view(np.uint32), ref.reshape(-1).view(np.uint32), err_msg=name)
    got = m.tensor(1000, "embed", c.vocab * c.hidden)
    np.testing.assert_array_equal(got.view(np.uint32), w["embed"].reshape(-1).view(np.uint32))
    m.close()


def test_teacher_forced_decode_matches_oracle_across_kv_slices():
    c = small()
    m, o = Qwen2(c), qo.Model(ocfg(c))
    tok, checked = 5, 0
    for pos in range(140):                      # crosses the 128-position slice boundary
        want, ref = o.step(tok, pos, return_logits=True)
        got = int(m.infer([tok], [pos])[0])
        if pos < 8 or pos in (127, 128, 129, 139):
            logits = m.logits()[0]
            assert rel(logits, ref) < TOL, f"pos {pos}"
            top2 = np.sort(ref)[-2:]
            if top2[1] - top2[0] > 4 * TOL * np.abs(ref).max():
                assert got == want, f"pos {pos}"
                checked += 1
        tok = want
    assert checked > 0
    m.close()


def test_device_feedback_equals_step_by_step_for_128_tokens():
    c = small()
    a, b = Qwen2(c), Qwen2(c)
    tok, seq = 9, []
    for pos in range(128):
        tok = int(a.infer([tok], [pos])[0])
        seq.append(tok)
    b.prep([9], [0])
    assert b.decode(128)[:, 0].tolist() == seq
    a.close(), b.close()


def test_one_step_at_qwen2_0_5b_shapes():
    c = Qwen2Config(layers=2, max_seq=64, seed=1)          # hidden 896, inter 4864, 14/2 heads, vocab 151936
    m, o = Qwen2(c), qo.Model(ocfg(c))
    tok = 1234
    for pos in range(3):
        want, ref = o.step(tok, pos, return_logits=True)
        m.infer([tok], [pos])
        assert rel(m.logits()[0], ref) < TOL
        tok = want
    m.close()


def test_128_free_running_greedy_steps_at_config_1_widths():
    """benchmark config 1's protocol (32-token prompt, then 128 greedy tokens with the argmax fed back on the
    device) at the Qwen2-0.5B widths with 4 of the 24 layers, against the C oracle fed the device's tokens: the
    oracle must pick the same token wherever its top-2 margin exceeds twice the logit bound, and a second
    instance replays the sequence step by step to check the bound itself at every step."""
    from oracle import c_oracle
    GUARD = 1e-4
    c = Qwen2Config(layers=4, max_seq=176, seed=2)
    a, b, o = Qwen2(c), Qwen2(c), c_oracle.Qwen2C(ocfg(c))
    prompt = np.random.default_rng(1000).integers(0, c.vocab, size=32).tolist()
    for pos in range(31):
        a.infer([prompt[pos]], [pos])
        b.infer([prompt[pos]], [pos])
        o.step(prompt[pos], pos)
    a.prep([prompt[31]], [31])
    seq = a.decode(128)[:, 0].tolist()
    tok, guarded, margins = prompt[31], 0, []
    for i in range(128):
        pos = 31 + i
        want, ref = o.step(tok, pos, return_logits=True)
        assert int(b.infer([tok], [pos])[0]) == seq[i]
        assert rel(b.logits()[0], ref) < GUARD, f"pos {pos}"
        top2 = np.sort(ref)[-2:]
        margins.append(float(top2[1] - top2[0]) / float(np.abs(ref).max()))
        if margins[-1] > 2 * GUARD:
            assert seq[i] == want, f"pos {pos}: margin {margins[-1]:.2e}"
            guarded += 1
        tok = seq[i]
    print(f"top-2 margins / max|logit|: min {min(margins):.2e}, median {np.median(margins):.2e}; {guarded}/128 steps decided")
    assert guarded >= 110
    a.close(), b.close(), o.close()


def test_steps_past_the_end_of_the_cache_are_refused():
    c = small(max_seq=16)
    m = Qwen2(c)
    m.prep([1], [14])
    assert m.decode(2).shape == (2, 1)
    with pytest.raises(RuntimeError, match="out of range"):
        m.decode(1)
    m.prep([1], [10])
    with pytest.raises(RuntimeError, match="out of range"):
        m.decode(7)
    m.base.execute(m.art.main, c.header())       # load again on a loaded instance
    assert m.infer([1], [0]).shape == (1,)
    m.close()


def test_weights_from_a_flat_file_replace_the_seeded_ones(tmp_path):
    """The reference's flat f32 weight file (tools/qwen2_convert.py:12-28) written with random tensors, loaded through the
    `setTensor` stage: the device reads back exactly what the file holds, and decodes like the oracle given the same
    tensors (not like the seeded model)."""
    from base_b200 import convert as cv
    c = small(layers=2, vocab=320)
    rng = np.random.default_rng(17)
    flat = {(n, l): (rng.standard_normal(shape) * 0.05).astype(np.float32) for n, l, shape in cv.qwen2_flat_layout(c)}
    for key in list(flat):
        if key[0] in ("ln1", "ln2", "lnf"):
            flat[key] = (flat[key] + 1).astype(np.float32)
    flat[("lm_head", None)] = flat[("embed", None)]
    path = tmp_path / "qwen2.bin"
    cv.write_qwen2_flat(path, c, flat)
    m = Qwen2(c)
    seeded = int(m.infer([5], [0])[0])
    seeded_logits = m.logits()[0].copy()
    cv.load_qwen2_flat(m, path)
    stage = {(l, k): np.asarray(a) for l, k, a in cv.qwen2_stage_tensors(c, cv.read_qwen2_flat(path, c))}
    np.testing.assert_array_equal(m.tensor(1, "wgu", stage[(1, "wgu")].size), stage[(1, "wgu")].ravel())
    np.testing.assert_array_equal(m.tensor(1000, "embed", stage[(1000, "embed")].size), stage[(1000, "embed")].ravel())
    w = {"embed": stage[(1000, "embed")], "lnf": stage[(1000, "lnf")],
         "layers": [{k: stage[(l, k)] for k in ("ln1", "wqkv", "bqkv", "wo", "ln2", "wgu", "wdn")} for l in range(c.layers)]}
    o = qo.Model(ocfg(c), w)
    tok = 5
    for pos in range(6):
        want, ref = o.step(tok, pos, return_logits=True)
        got = int(m.infer([tok], [pos])[0])
        logits = m.logits()[0]
        assert rel(logits, ref) < TOL, f"pos {pos}: {rel(logits, ref)}"
        top2 = np.sort(ref)[-2:]
        if top2[1] - top2[0] > 4 * TOL * np.abs(ref).max():
            assert got == want
        if pos == 0:
            assert rel(logits, seeded_logits) > 1e-2          # these are not the seeded model's logits any more
        tok = want
    with pytest.raises(RuntimeError, match="wrong size"):
        m.set_tensor(0, "ln1", np.zeros(3, np.float32))
    with pytest.raises(RuntimeError, match="no such tensor"):
        m.base.execute(m.art.extras["setTensor"], b"\x07\x00\x00\x00\x09\x00\x00\x00" + b"\0" * 4)
    m.close()
    del seeded


def test_on_disk_mode_decodes_exactly_like_the_resident_model(tmp_path):
    """The reference's second storage strategy (one layer's weights and one K/V pair on the device, the layers streamed
    from the weight file and the cache kept in a file, Qwen2OnDiskAlgorithm.lean:18-42) must give byte-identical output
    (applications/qwen2/tests/golden_cli.rs:1-8): same tokens and bit-equal logits as the resident model, fed step by
    step and with the argmax fed back on the device."""
    from base_b200 import convert as cv
    from base_b200.qwen2 import ON_DISK
    c = small(layers=3, vocab=320, max_seq=40)
    m = Qwen2(c)
    QD, KVD, F = c.n_q * 64, c.n_kv * 64, c.inter
    flat = {("embed", None): m.tensor(1000, "embed", c.vocab * c.hidden).reshape(c.vocab, c.hidden),
            ("lnf", None): m.tensor(1000, "lnf", c.hidden)}
    flat[("lm_head", None)] = flat[("embed", None)]
    for l in range(c.layers):
        wqkv = m.tensor(l, "wqkv", (QD + 2 * KVD) * c.hidden).reshape(QD + 2 * KVD, c.hidden)
        bqkv = m.tensor(l, "bqkv", QD + 2 * KVD)
        wgu = m.tensor(l, "wgu", 2 * F * c.hidden).reshape(2 * F, c.hidden)
        flat.update({("ln1", l): m.tensor(l, "ln1", c.hidden), ("wq", l): wqkv[:QD], ("wk", l): wqkv[QD:QD + KVD],
                     ("wv", l): wqkv[QD + KVD:], ("bq", l): bqkv[:QD], ("bk", l): bqkv[QD:QD + KVD], ("bv", l): bqkv[QD + KVD:],
                     ("wo", l): m.tensor(l, "wo", c.hidden * QD).reshape(c.hidden, QD), ("ln2", l): m.tensor(l, "ln2", c.hidden),
                     ("wgate", l): wgu[:F], ("wup", l): wgu[F:],
                     ("wdn", l): m.tensor(l, "wdn", c.hidden * F).reshape(c.hidden, F)})
    wpath, kvpath = tmp_path / "w.bin", tmp_path / "kv.bin"
    cv.write_qwen2_flat(wpath, c, flat)
    import dataclasses
    d = Qwen2(dataclasses.replace(c, flags=c.flags | ON_DISK))
    with pytest.raises(RuntimeError, match="openFiles has not run"):
        d.infer([5], [0])
    d.open_files(str(wpath), str(kvpath))
    assert kvpath.stat().st_size == c.layers * 2 * c.n_kv * c.max_seq * 64 * 4
    tok = 5
    for pos in range(5):
        a, b = int(m.infer([tok], [pos])[0]), int(d.infer([tok], [pos])[0])
        assert a == b
        np.testing.assert_array_equal(m.logits(), d.logits())
        tok = a
    m.prep([tok], [5])
    d.prep([tok], [5])
    np.testing.assert_array_equal(m.decode(6), d.decode(6))                      # device feedback, cache rows through the file
    kv = np.fromfile(kvpath, dtype="<f4").reshape(c.layers, 2, c.n_kv, c.max_seq, 64)
    assert np.abs(kv[:, :, :, :11]).max(axis=-1).min() > 0 and not kv[:, :, :, 11:].any()    # 11 positions written, the rest untouched
    other = Qwen2(dataclasses.replace(c, layers=2, flags=c.flags | ON_DISK))
    with pytest.raises(RuntimeError, match="size does not match"):
        other.open_files(str(wpath), str(kvpath))
    other.close()
    m.close()
    d.close()
