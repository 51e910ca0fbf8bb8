"""MXFP4 quantiser, flat weight file and the Hugging Face name map of base_b200/convert.py (CPU)."""
import numpy as np
import pytest

from base_b200 import convert as cv
from base_b200.gptoss import GptOssConfig
from oracle import moe_oracle as mo
from oracle import synth


def tiny_cfg(**kw):
    base = dict(layers=2, hidden=128, inter=192, experts=8, top_k=4, n_q=8, n_kv=2, vocab=512, window=8, max_seq=64, seed=1)
    base.update(kw)
    return GptOssConfig(**base)


def random_weights(c: GptOssConfig, seed=3) -> dict:
    """Oracle-style weights: bf16 tensors as the f32 values they hold, experts quantised by the converter."""
    r = np.random.default_rng(seed)
    H, I, E, QD, QKV = c.hidden, c.inter, c.experts, c.n_q * 64, (c.n_q + 2 * c.n_kv) * 64

    def n(*shape, s=0.02):
        return (r.standard_normal(shape) * s).astype(np.float32)
    w = {"embed": synth.bf16_round(n(c.vocab, H)), "lm_head": synth.bf16_round(n(c.vocab, H)), "lnf": 1 + n(H), "layers": []}
    for l in range(c.layers):
        guc, gus = cv.quantize_mxfp4(n(E, 2 * I, H, s=0.05))
        dnc, dns = cv.quantize_mxfp4(n(E, H, I, s=0.05))
        w["layers"].append({"ln1": 1 + n(H), "wqkv": synth.bf16_round(n(QKV, H)), "bqkv": n(QKV), "sinks": n(c.n_q, s=1.0),
                            "wo": synth.bf16_round(n(H, QD)), "bo": n(H), "ln2": 1 + n(H), "Wr": n(E, H, s=0.5), "br": n(E, s=0.01),
                            "gu_codes": guc, "gu_scales": gus, "gu_bias": n(E, 2 * I, s=0.01),
                            "dn_codes": dnc, "dn_scales": dns, "dn_bias": n(E, H, s=0.01),
                            "top_k": c.top_k, "alpha": c.alpha, "limit": c.limit, "window": c.window if l % 2 == 0 else 0})
    return w


def test_quantiser_rounds_to_the_nearest_e2m1_value_and_inverts_exactly():
    r = np.random.default_rng(0)
    w = (r.standard_normal((7, 96)) * np.exp(r.standard_normal((7, 1)) * 3)).astype(np.float32)
    codes, scales = cv.quantize_mxfp4(w)
    assert codes.shape == (7, 48) and scales.shape == (7, 3) and scales.min() >= 1 and scales.max() <= 254
    deq = cv.dequantize_mxfp4(codes, scales)
    np.testing.assert_array_equal(deq.view(np.uint32), mo.mx_dequant(codes, scales).view(np.uint32))   # the oracle's table and layout
    # error: the grid is at most 2 scale units wide at the top (4 .. 6) and the largest magnitude lies in [4, 8) scale units
    step = np.ldexp(np.float32(1.0), scales.astype(np.int32) - 127)[..., None]
    err = np.abs(deq - w).reshape(7, 3, 32)
    assert (err <= step * 2.0 + 1e-12).all()                 # 2 steps only where a value in (6, 8) saturates at 6
    assert (err <= np.maximum(np.abs(w).reshape(7, 3, 32) * 0.25, step * 0.25) + 1e-12).all()
    # values that are exactly representable come back bit for bit
    c2, s2 = cv.quantize_mxfp4(deq)
    np.testing.assert_array_equal(cv.dequantize_mxfp4(c2, s2), deq)
    # ties go to the even code: 2.5 (between 2 and 3) -> 2, 5 (between 4 and 6) -> 4, 0.25 -> 0, 0.75 -> 1
    t = np.zeros((1, 32), dtype=np.float32)
    t[0, :5] = [6.0, 2.5, 5.0, 0.25, 0.75]
    ct, st = cv.quantize_mxfp4(t)
    assert st[0, 0] == 127 and cv.dequantize_mxfp4(ct, st)[0, :5].tolist() == [6.0, 2.0, 4.0, 0.0, 1.0]
    z, sz = cv.quantize_mxfp4(np.zeros((1, 32), dtype=np.float32))
    assert not z.any() and cv.dequantize_mxfp4(z, sz).max() == 0.0


def test_weight_file_round_trip_and_header(tmp_path):
    c = tiny_cfg()
    w = random_weights(c)
    p = tmp_path / "w.bin"
    cv.write_checkpoint(p, c, w)
    fc = cv.read_config(p)
    assert (fc.layers, fc.hidden, fc.experts, fc.vocab, fc.n_q) == (c.layers, c.hidden, c.experts, c.vocab, c.n_q)
    raw = np.fromfile(p, dtype=np.uint8)
    H, V = c.hidden, c.vocab
    emb = raw[128:128 + V * H * 2].view("<u2")
    np.testing.assert_array_equal(emb, synth.f32_to_bf16_bits(w["embed"].reshape(-1)))
    tail = raw[-V * H * 2:].view("<u2")
    np.testing.assert_array_equal(tail, synth.f32_to_bf16_bits(w["lm_head"].reshape(-1)))
    sizes = cv._shapes(c)
    per_layer = sum(int(np.prod(sizes[k])) * (2 if dt == "bf16" else np.dtype(dt).itemsize) for k, _, dt in cv._LAYER)
    assert raw.size == 128 + 2 * V * H * 2 + c.layers * per_layer + H * 4
    with pytest.raises(ValueError):
        (tmp_path / "bad.bin").write_bytes(b"\0" * 256)
        cv.read_config(tmp_path / "bad.bin")


def test_hugging_face_names_map_onto_the_weights_dict():
    c = tiny_cfg(layers=1)
    w = random_weights(c)
    ly = w["layers"][0]
    QD, KVD = c.n_q * 64, c.n_kv * 64
    sd = {"model.embed_tokens.weight": w["embed"], "model.norm.weight": w["lnf"], "lm_head.weight": w["lm_head"]}
    p, a, m = "model.layers.0.", "model.layers.0.self_attn.", "model.layers.0.mlp."
    sd.update({p + "input_layernorm.weight": ly["ln1"], p + "post_attention_layernorm.weight": ly["ln2"],
               a + "q_proj.weight": ly["wqkv"][:QD], a + "k_proj.weight": ly["wqkv"][QD:QD + KVD], a + "v_proj.weight": ly["wqkv"][QD + KVD:],
               a + "q_proj.bias": ly["bqkv"][:QD], a + "k_proj.bias": ly["bqkv"][QD:QD + KVD], a + "v_proj.bias": ly["bqkv"][QD + KVD:],
               a + "sinks": ly["sinks"], a + "o_proj.weight": ly["wo"], a + "o_proj.bias": ly["bo"],
               m + "router.weight": ly["Wr"], m + "router.bias": ly["br"],
               m + "experts.gate_up_proj_blocks": ly["gu_codes"].reshape(c.experts, 2 * c.inter, c.hidden // 32, 16),
               m + "experts.gate_up_proj_scales": ly["gu_scales"], m + "experts.gate_up_proj_bias": ly["gu_bias"],
               m + "experts.down_proj_blocks": ly["dn_codes"].reshape(c.experts, c.hidden, c.inter // 32, 16),
               m + "experts.down_proj_scales": ly["dn_scales"], m + "experts.down_proj_bias": ly["dn_bias"]})
    got = cv.from_hf_state_dict(sd, c)
    for k in ("embed", "lnf", "lm_head"):
        np.testing.assert_array_equal(got[k], w[k])
    for k, _, _ in cv._LAYER:
        np.testing.assert_array_equal(got["layers"][0][k], ly[k], err_msg=k)


# ---- Qwen2: the reference's flat f32 weight file ---------------------------------------------------------------------
def qwen2_tiny():
    from base_b200.qwen2 import Qwen2Config
    return Qwen2Config(layers=2, hidden=64, inter=128, n_q=2, n_kv=1, vocab=96, max_seq=32)


def qwen2_random_flat(c, seed=9, tie=True):
    rng = np.random.default_rng(seed)
    flat = {(n, l): rng.standard_normal(shape).astype(np.float32) * np.float32(0.05) for n, l, shape in cv.qwen2_flat_layout(c)}
    for key in list(flat):
        if key[0] in ("ln1", "ln2", "lnf"):
            flat[key] = (flat[key] + 1).astype(np.float32)
    if tie:
        flat[("lm_head", None)] = flat[("embed", None)]
    return flat


def test_qwen2_flat_file_order_sizes_and_round_trip(tmp_path):
    from base_b200.qwen2 import QWEN2_0_5B
    c = qwen2_tiny()
    names = [n for n, _, _ in cv.qwen2_flat_layout(c)]
    per_layer = ["ln1", "wq", "bq", "wk", "bk", "wv", "bv", "wo", "ln2", "wgate", "wup", "wdn"]      # the converter's write order
    assert names == ["embed"] + per_layer * c.layers + ["lnf", "lm_head"]
    assert cv.qwen2_flat_bytes(QWEN2_0_5B) == 4 * (2 * 151936 * 896 + 896 + 24 * (
        2 * 896 + 896 * 896 + 896 + 2 * (128 * 896 + 128) + 896 * 896 + 3 * 4864 * 896))
    flat = qwen2_random_flat(c)
    p = tmp_path / "w.bin"
    cv.write_qwen2_flat(p, c, flat)
    assert p.stat().st_size == cv.qwen2_flat_bytes(c)
    back = cv.read_qwen2_flat(p, c)
    for key, a in flat.items():
        np.testing.assert_array_equal(back[key], a)
    raw = np.fromfile(p, dtype="<f4")
    np.testing.assert_array_equal(raw[:c.vocab * c.hidden], flat[("embed", None)].ravel())             # first in the file
    np.testing.assert_array_equal(raw[-c.vocab * c.hidden:], flat[("lm_head", None)].ravel())          # last
    with open(p, "ab") as f:
        f.write(b"\0\0\0\0")
    with pytest.raises(ValueError):
        cv.read_qwen2_flat(p, c)


def test_qwen2_stage_tensors_concatenate_projections_and_refuse_an_untied_head():
    c = qwen2_tiny()
    flat = qwen2_random_flat(c)
    got = {(l, k): a for l, k, a in cv.qwen2_stage_tensors(c, flat)}
    assert set(k for _, k in got) == {"embed", "lnf", "ln1", "wqkv", "bqkv", "wo", "ln2", "wgu", "wdn"}
    qd, kvd = c.n_q * 64, c.n_kv * 64
    w = got[(1, "wqkv")]
    assert w.shape == (qd + 2 * kvd, c.hidden)
    np.testing.assert_array_equal(w[:qd], flat[("wq", 1)])
    np.testing.assert_array_equal(w[qd:qd + kvd], flat[("wk", 1)])
    np.testing.assert_array_equal(w[qd + kvd:], flat[("wv", 1)])
    np.testing.assert_array_equal(got[(0, "wgu")][:c.inter], flat[("wgate", 0)])
    np.testing.assert_array_equal(got[(0, "wgu")][c.inter:], flat[("wup", 0)])
    np.testing.assert_array_equal(got[(0, "bqkv")], np.concatenate([flat[("bq", 0)], flat[("bk", 0)], flat[("bv", 0)]]))
    with pytest.raises(ValueError):
        list(cv.qwen2_stage_tensors(c, qwen2_random_flat(c, tie=False)))


def test_qwen2_hf_names_map_to_the_file():
    c = qwen2_tiny()
    flat = qwen2_random_flat(c)
    hf = {"model.embed_tokens.weight": flat[("embed", None)], "model.norm.weight": flat[("lnf", None)]}
    names = dict(ln1="input_layernorm.weight", wq="self_attn.q_proj.weight", bq="self_attn.q_proj.bias", wk="self_attn.k_proj.weight",
                 bk="self_attn.k_proj.bias", wv="self_attn.v_proj.weight", bv="self_attn.v_proj.bias", wo="self_attn.o_proj.weight",
                 ln2="post_attention_layernorm.weight", wgate="mlp.gate_proj.weight", wup="mlp.up_proj.weight", wdn="mlp.down_proj.weight")
    for l in range(c.layers):
        for k, n in names.items():
            hf[f"model.layers.{l}.{n}"] = flat[(k, l)]
    back = cv.qwen2_flat_from_hf_state_dict(hf, c)                  # no lm_head.weight: tied to the embedding
    assert set(back) == set(flat)
    for key in flat:
        np.testing.assert_array_equal(back[key], flat[key])
