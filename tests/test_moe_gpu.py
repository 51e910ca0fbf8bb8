"""Parity of the CUDA MoE path against the oracle, through Base/execute_into
(i.e. through the C-ABI).  Bit-exact: dequantised values, top-k indices, the
token permutation.  Tolerance: FFN output max|d|/max|ref| <= 1e-4 with f32
activations (hi+lo split), <= 1e-2 in the one-column (bf16-class) mode."""
import numpy as np
import pytest

from base_b200.moe import MoeConfig, MoeFfn, make_moe_params
from oracle import moe_oracle as mo

pytestmark = pytest.mark.gpu

TOL_F32 = 1e-4
TOL_HALF = 1e-2
PDL, CKPT_LAYOUT, ONE_COLUMN, NO_RINGS = 1, 2, 4, 8


def rel(got, ref):
    return float(np.abs(got - ref).max() / max(np.abs(ref).max(), 1e-30))


def hf_moe_inputs():
    H, I, E, k, T = 64, 96, 8, 4, 5
    r = np.random.default_rng(202)
    p = {
        "Wr": (r.standard_normal((E, H)) * 0.5).astype(np.float32),
        "br": (r.standard_normal(E) * 0.1).astype(np.float32),
        "gu_codes": r.integers(0, 256, size=(E, 2 * I, H // 2), dtype=np.uint8),
        "gu_scales": r.integers(121, 126, size=(E, 2 * I, H // 32), dtype=np.uint8),
        "gu_bias": (r.standard_normal((E, 2 * I)) * 0.5).astype(np.float32),
        "dn_codes": r.integers(0, 256, size=(E, H, I // 2), dtype=np.uint8),
        "dn_scales": r.integers(121, 126, size=(E, H, I // 32), dtype=np.uint8),
        "dn_bias": (r.standard_normal((E, H)) * 0.1).astype(np.float32),
        "top_k": k, "alpha": 1.702, "limit": 7.0,
    }
    x = (r.standard_normal((T, H)) * 1.5).astype(np.float32)
    return p, x


def check_layer(cfg, p, x, m, tol=TOL_F32):
    y = m.forward(x)
    idx, w = m.topk()
    ry, ridx, rw, rlogits, racts = mo.moe_ffn(x, p, return_all=True)
    assert rel(m.logits(), rlogits) < 1e-5
    margin = mo.topk_margin(rlogits, cfg.top_k)
    safe = margin > 1e-4 * np.abs(rlogits).max()
    assert safe.any()
    np.testing.assert_array_equal(idx[safe], ridx[safe])
    np.testing.assert_allclose(w[safe], rw[safe], atol=5e-6)
    assert rel(m.acts()[safe], racts[safe]) < tol
    assert rel(y[safe], ry[safe]) < tol
    if m.tiled():
        # the permutation is integer work: bit-exact given the device's own indices
        want = mo.route_tables(idx, cfg.experts)
        got = m.route()
        assert got["n_active"] == want["n_active"]
        for k in ("count", "offset", "active", "perm"):
            np.testing.assert_array_equal(got[k], want[k], err_msg=k)
    return y, ry, ridx, rw


@pytest.mark.parametrize("flags", [0, NO_RINGS, CKPT_LAYOUT])
def test_small_layer_tokens_1_to_8(flags):
    cfg = MoeConfig(hidden=128, inter=192, experts=8, top_k=4)
    p = make_moe_params(cfg, seed=3)
    p["Wr"] *= 25
    r = np.random.default_rng(4)
    m = MoeFfn(cfg, p, max_tokens=16, flags=flags)
    assert m.tiled() == (flags != CKPT_LAYOUT)
    for T in (1, 2, 5, 8, 16):
        check_layer(cfg, p, r.standard_normal((T, cfg.hidden)).astype(np.float32), m)
    m.close()


def test_shapes_the_tiled_layout_cannot_take_use_the_checkpoint_layout():
    cfg = MoeConfig(hidden=64, inter=96, experts=8, top_k=4)      # inter % 64 != 0
    p = make_moe_params(cfg, seed=3)
    p["Wr"] *= 25
    m = MoeFfn(cfg, p)
    assert not m.tiled()
    check_layer(cfg, p, np.random.default_rng(5).standard_normal((3, 64)).astype(np.float32), m)
    m.close()


@pytest.mark.parametrize("flags", [0, NO_RINGS])
def test_many_tokens_per_expert_and_uneven_routing(flags):
    # 40 tokens over 8 experts with a skewed router: some experts get > 8
    # assignments (several MMA passes), some may get none.
    cfg = MoeConfig(hidden=128, inter=128, experts=8, top_k=2)
    p = make_moe_params(cfg, seed=13, skew=0.5)
    p["Wr"] *= 10
    x = np.random.default_rng(14).standard_normal((40, cfg.hidden)).astype(np.float32)
    m = MoeFfn(cfg, p, max_tokens=64, flags=flags)
    check_layer(cfg, p, x, m)
    counts = m.route()["count"]
    assert counts.max() > 8 and counts.sum() == 80
    m.close()


@pytest.mark.parametrize("rings", [0, NO_RINGS])
def test_one_column_mode_is_within_bf16_tolerance(rings):
    cfg = MoeConfig(hidden=128, inter=192, experts=8, top_k=4)
    p = make_moe_params(cfg, seed=3)
    p["Wr"] *= 25
    x = np.random.default_rng(6).standard_normal((9, cfg.hidden)).astype(np.float32)
    m = MoeFfn(cfg, p, max_tokens=16, flags=ONE_COLUMN | rings)
    check_layer(cfg, p, x, m, tol=TOL_HALF)
    m.close()


def test_transformers_fixture_through_gpu(golden):
    g = np.load(golden / "hf_gptoss_moe.npz")
    p, x = hf_moe_inputs()
    cfg = MoeConfig(hidden=64, inter=96, experts=8, top_k=4)
    m = MoeFfn(cfg, p)
    y = m.forward(x)
    idx, w = m.topk()
    np.testing.assert_array_equal(idx, g["indices"])
    np.testing.assert_allclose(w, g["scores"], atol=5e-6)
    assert rel(y, g["y"]) < TOL_F32
    m.close()


def test_dequantised_values_bit_exact_both_layouts():
    cfg = MoeConfig(hidden=192, inter=64, experts=3, top_k=2)
    p = make_moe_params(cfg, seed=9)
    p["gu_codes"][1, 0, :16] = (np.arange(16) * 17).astype(np.uint8)     # every code value
    p["gu_scales"][1, 1, :] = [127, 200, 60, 1, 254, 2]                  # extreme but regular scales
    for flags in (0, CKPT_LAYOUT):
        m = MoeFfn(cfg, p, flags=flags)
        assert m.tiled() == (flags == 0)
        for which, codes, scales in ((0, p["gu_codes"], p["gu_scales"]), (1, p["dn_codes"], p["dn_scales"])):
            for e in range(cfg.experts):
                n = min(codes.shape[1], 64)
                got = m.dequant(which, e, 0, n)
                want = mo.mx_dequant(codes[e, :n], scales[e, :n])
                np.testing.assert_array_equal(got.view(np.uint32), want.view(np.uint32))
        m.close()


def test_scale_bytes_0_and_255_fall_back_and_stay_bit_exact():
    cfg = MoeConfig(hidden=128, inter=64, experts=2, top_k=1)
    p = make_moe_params(cfg, seed=10)
    p["dn_scales"][1, 5, :] = [0, 255]        # 2^-127 (f32 subnormal) and NaN
    m = MoeFfn(cfg, p)
    assert not m.tiled()
    got = m.dequant(1, 1, 0, 16)
    want = mo.mx_dequant(p["dn_codes"][1, :16], p["dn_scales"][1, :16])
    np.testing.assert_array_equal(got.view(np.uint32) & 0xff800000, want.view(np.uint32) & 0xff800000)
    ok = ~np.isnan(want)
    np.testing.assert_array_equal(got[ok], want[ok])
    assert np.isnan(got[~ok]).all()
    m.close()


def test_topk_ties_and_order():
    cfg = MoeConfig(hidden=64, inter=64, experts=8, top_k=4)
    p = make_moe_params(cfg, seed=1)
    p["Wr"][:] = 0
    p["br"][:] = np.array([1, 3, 3, 2, 3, -1, 0, 2], dtype=np.float32)   # ties: 1,2,4 then 3,7
    m = MoeFfn(cfg, p)
    m.forward(np.ones((2, 64), dtype=np.float32))
    idx, w = m.topk()
    assert idx.tolist() == [[1, 2, 4, 3]] * 2
    ridx, rw = mo.topk_softmax(np.tile(p["br"], (2, 1)), 4)
    np.testing.assert_array_equal(idx, ridx)
    np.testing.assert_allclose(w, rw, atol=1e-6)
    m.close()


def test_different_expert_set_gives_a_different_answer():
    # the reference's non-vacuity guard, applications/ten-qwen/moe.py:88-95
    cfg = MoeConfig(hidden=64, inter=64, experts=8, top_k=2)
    p = make_moe_params(cfg, seed=21)
    p["Wr"] *= 25
    x = np.random.default_rng(22).standard_normal((1, 64)).astype(np.float32)
    m = MoeFfn(cfg, p)
    y = m.forward(x)
    idx, w = m.topk()
    others = [e for e in range(cfg.experts) if e not in set(idx[0].tolist())][:2]
    alt = np.zeros(64, dtype=np.float32)
    for j, e in enumerate(others):
        o, _ = mo.expert_ffn(x[0], mo.mx_dequant(p["gu_codes"][e], p["gu_scales"][e]), p["gu_bias"][e],
                             mo.mx_dequant(p["dn_codes"][e], p["dn_scales"][e]), p["dn_bias"][e])
        alt += w[0, j] * o
    assert rel(alt, y[0]) > 1e-2
    m.close()


@pytest.mark.parametrize("layout", [0, NO_RINGS, CKPT_LAYOUT])
def test_pdl_launch_is_bit_identical_and_repeatable(layout):
    # a scheduling change must not change results (cf. the reference's graph
    # replay check, applications/ten-qwen/profile.py:67-70)
    cfg = MoeConfig(hidden=128, inter=128, experts=8, top_k=4)
    p = make_moe_params(cfg, seed=31)
    x = np.random.default_rng(32).standard_normal((3, 128)).astype(np.float32)
    a = MoeFfn(cfg, p, flags=layout)
    b = MoeFfn(cfg, p, flags=layout | PDL)
    ya, yb = a.forward(x), b.forward(x)
    np.testing.assert_array_equal(ya.view(np.uint32), yb.view(np.uint32))
    b.stack(5)
    np.testing.assert_array_equal(b.infer().view(np.uint32), ya.view(np.uint32))
    a.close(), b.close()


def test_stage_errors_are_reported():
    cfg = MoeConfig(hidden=64, inter=64, experts=4, top_k=2)
    p = make_moe_params(cfg, seed=2)
    m = MoeFfn(cfg, p, max_tokens=2)
    with pytest.raises(RuntimeError, match="max_tokens"):
        m.prep(np.zeros((3, 64), dtype=np.float32))
    with pytest.raises(RuntimeError, match="bad magic"):        # a bad request leaves the loaded instance as it is
        m.base.execute(m.art.main, b"\0" * 64)
    m.prep(np.zeros((1, 64), dtype=np.float32))
    with pytest.raises(RuntimeError, match="out must be"):
        m.base.execute_into(m.art.extras["infer"], b"", bytearray(8))
    m.close()


@pytest.mark.parametrize("flags", [PDL, NO_RINGS, CKPT_LAYOUT])
def test_gpt_oss_20b_layer_config0(flags):
    # benchmark config 0: hidden 2880, inter 2880, 32 experts, top-4, 1 decode token.
    cfg = MoeConfig()
    p = make_moe_params(cfg, seed=0)
    x = np.random.default_rng(1).standard_normal((1, cfg.hidden)).astype(np.float32)
    m = MoeFfn(cfg, p, max_tokens=4, flags=flags)
    y, ry, ridx, rw = check_layer(cfg, p, x, m)
    # bit-exact dequant at full size on rows at both ends of the matrix
    for which, codes, scales in ((0, p["gu_codes"], p["gu_scales"]), (1, p["dn_codes"], p["dn_scales"])):
        e = int(ridx[0, 0])
        for row0 in (0, codes.shape[1] - 64):
            got = m.dequant(which, e, row0, 64)
            want = mo.mx_dequant(codes[e, row0:row0 + 64], scales[e, row0:row0 + 64])
            np.testing.assert_array_equal(got.view(np.uint32), want.view(np.uint32))
    # SwiGLU rules out linearity checks; idempotence holds:
    y2 = m.infer()
    np.testing.assert_array_equal(y.view(np.uint32), y2.view(np.uint32))
    # 3 tokens reuse the same weights
    x3 = np.random.default_rng(2).standard_normal((3, cfg.hidden)).astype(np.float32)
    check_layer(cfg, p, x3, m)
    m.close()


BLOCK_SCALED = 64


@pytest.mark.timeout(180, method="thread")
@pytest.mark.parametrize("hidden,inter,experts", [(128, 192, 8), (256, 64, 8), (576, 320, 16)])
def test_block_scaled_tensor_core_path_small_layers(hidden, inter, experts):
    """One-token calls with flags bit 6 run both expert matrices on tcgen05.mma kind::mxf4
    (codes and scales as stored, activations as radix-8 E2M1 digits); other token counts
    of the same instance take the streaming kernels.  Same tolerance as the f32 path."""
    cfg = MoeConfig(hidden=hidden, inter=inter, experts=experts, top_k=4)
    p = make_moe_params(cfg, seed=hidden + inter)
    p["Wr"] *= 25
    r = np.random.default_rng(hidden)
    m = MoeFfn(cfg, p, max_tokens=8, flags=PDL | BLOCK_SCALED)
    for T in (1, 1, 3, 1):
        check_layer(cfg, p, r.standard_normal((T, cfg.hidden)).astype(np.float32), m)
    # activations spanning many binades inside one block
    x = (r.standard_normal((1, cfg.hidden)) * np.exp2(r.integers(-20, 8, size=(1, cfg.hidden)))).astype(np.float32)
    check_layer(cfg, p, x, m)
    m.close()


@pytest.mark.timeout(180, method="thread")
def test_block_scaled_tensor_core_path_config0():
    cfg = MoeConfig()
    p = make_moe_params(cfg, seed=0)
    x = np.random.default_rng(1).standard_normal((1, cfg.hidden)).astype(np.float32)
    m = MoeFfn(cfg, p, max_tokens=4, flags=PDL | BLOCK_SCALED)
    y, ry, ridx, rw = check_layer(cfg, p, x, m)
    y2 = m.infer()
    np.testing.assert_array_equal(y.view(np.uint32), y2.view(np.uint32))
    m.close()
