"""Weights on disk for the `native:gptoss` stage program: an MXFP4 quantiser, a flat weight file and its loader.

The reference ships `tools/qwen2_convert.py` (HF safetensors -> ONE flat little-endian file of f32 tensors in a fixed
order, tools/qwen2_convert.py:12-28, 101-141) and streams that file to the device tensor by tensor
(lean/algorithms/Qwen2Common.lean:503-515).  The same shape here for gpt-oss:

    file = [128-byte GptOssConfig.header()]
           embed bf16 [V][H]
           per layer: ln1 f32[H] | wqkv bf16 [QKV][H] (q rows, then k, then v) | bqkv f32[QKV] | sinks f32[NQ] |
                      wo bf16 [H][QD] | bo f32[H] | ln2 f32[H] | router f32 [E][H] | router bias f32[E] |
                      gate_up codes u8 [E][2I][H/2] | gate_up scales u8 [E][2I][H/32] | gate_up bias f32 [E][2I] |
                      down codes u8 [E][H][I/2] | down scales u8 [E][H][I/32] | down bias f32 [E][H]
           lnf f32[H] | lm_head bf16 [V][H]

MXFP4 as this library fixes it (csrc/kernels/common.cuh; the reference specifies the element table only,
lean/lib/AlgorithmLib/ML/QuantMX.lean:56-74, 131-147): code = sign << 3 | index into {0, .5, 1, 1.5, 2, 3, 4, 6}, two
codes per byte with the EVEN element in the low nibble, one UE8M0 scale byte per 32 elements (2^(byte - 127)),
gate/up rows interleaved (row 2i = gate_i, row 2i + 1 = up_i) — the layout of the Hugging Face gpt-oss checkpoints
(`*_blocks` [.., K/32, 16] is the same bytes as codes [.., K/2]).
"""
from __future__ import annotations

import struct
from pathlib import Path

import numpy as np

from .gptoss import KIND, GLOBAL_LAYER, GptOss, GptOssConfig, MAGIC

E2M1 = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=np.float32)
# midpoints between consecutive magnitudes; a value on a midpoint goes to the even code (round to nearest even)
_MID = (E2M1[:-1] + E2M1[1:]) / 2


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return ((u + np.uint64(0x7FFF) + ((u >> np.uint64(16)) & np.uint64(1))) >> np.uint64(16)).astype(np.uint16)


def quantize_mxfp4(w: np.ndarray):
    """f32 [..., K] (K % 32 == 0) -> (codes u8 [..., K/2], scales u8 [..., K/32]).

    Per 32-element block the scale is the power of two that puts the block's largest magnitude into [4, 8)
    (OCP MX: shared exponent = floor(log2(amax)) - 2, E2M1's largest exponent), elements are rounded to the nearest
    E2M1 value (ties to the even code) and saturate at 6."""
    w = np.ascontiguousarray(w, dtype=np.float32)
    K = w.shape[-1]
    assert K % 32 == 0
    blocks = w.reshape(*w.shape[:-1], K // 32, 32)
    amax = np.abs(blocks).max(axis=-1)
    exp = np.floor(np.log2(np.where(amax > 0, amax, 1.0))).astype(np.int32) - 2
    exp = np.clip(exp, 1 - 127, 254 - 127)                  # scale bytes 1..254 (0 and 255 are not used)
    scale = np.ldexp(np.float32(1.0), exp).astype(np.float32)
    mag = np.abs(blocks) / scale[..., None]
    idx = np.searchsorted(_MID, mag, side="left").astype(np.uint8)       # ties land on the lower index ...
    tie = np.isin(mag, _MID) & (idx % 2 == 1)                            # ... move them to the even code
    idx = np.where(tie, idx + 1, idx).astype(np.uint8)
    idx = np.minimum(idx, 7)
    code = (idx | (np.signbit(blocks).astype(np.uint8) << 3)).reshape(*w.shape[:-1], K)
    packed = (code[..., 0::2] | (code[..., 1::2] << 4)).astype(np.uint8)
    return packed, (exp + 127).astype(np.uint8)


def dequantize_mxfp4(codes: np.ndarray, scales: np.ndarray) -> np.ndarray:
    """The inverse map (exact): codes u8 [..., K/2], scales u8 [..., K/32] -> f32 [..., K]."""
    lo, hi = codes & 15, codes >> 4
    c = np.stack([lo, hi], axis=-1).reshape(*codes.shape[:-1], codes.shape[-1] * 2)
    v = E2M1[c & 7] * np.where(c & 8, np.float32(-1), np.float32(1))
    s = np.ldexp(np.float32(1.0), scales.astype(np.int32) - 127).astype(np.float32)
    return (v.reshape(*scales.shape, 32) * s[..., None]).reshape(v.shape).astype(np.float32)


# tensors of a layer in file order: (key in the weights dict, kind, dtype)
_LAYER = (("ln1", "ln1", "<f4"), ("wqkv", "wqkv", "bf16"), ("bqkv", "bqkv", "<f4"), ("sinks", "sinks", "<f4"),
          ("wo", "wo", "bf16"), ("bo", "bo", "<f4"), ("ln2", "ln2", "<f4"), ("Wr", "wr", "<f4"), ("br", "br", "<f4"),
          ("gu_codes", "gu_codes", "u1"), ("gu_scales", "gu_scales", "u1"), ("gu_bias", "gu_bias", "<f4"),
          ("dn_codes", "dn_codes", "u1"), ("dn_scales", "dn_scales", "u1"), ("dn_bias", "dn_bias", "<f4"))


def _shapes(c: GptOssConfig) -> dict:
    H, I, E, V = c.hidden, c.inter, c.experts, c.vocab
    QD, QKV = c.n_q * 64, (c.n_q + 2 * c.n_kv) * 64
    return {"embed": (V, H), "lm_head": (V, H), "lnf": (H,), "ln1": (H,), "wqkv": (QKV, H), "bqkv": (QKV,),
            "sinks": (c.n_q,), "wo": (H, QD), "bo": (H,), "ln2": (H,), "Wr": (E, H), "br": (E,),
            "gu_codes": (E, 2 * I, H // 2), "gu_scales": (E, 2 * I, H // 32), "gu_bias": (E, 2 * I),
            "dn_codes": (E, H, I // 2), "dn_scales": (E, H, I // 32), "dn_bias": (E, H)}


def _raw(a: np.ndarray, dtype: str) -> bytes:
    if dtype == "bf16":
        return f32_to_bf16_bits(np.asarray(a, dtype=np.float32)).astype("<u2").tobytes()
    return np.ascontiguousarray(a, dtype=dtype).tobytes()


def write_checkpoint(path, cfg: GptOssConfig, w: dict) -> None:
    """`w` as oracle-style dict: embed, lm_head, lnf, layers[l][ln1, wqkv, ..., dn_bias] (bf16 tensors given as f32)."""
    sh = _shapes(cfg)
    with open(path, "wb") as f:
        f.write(cfg.header())
        assert tuple(w["embed"].shape) == sh["embed"]
        f.write(_raw(w["embed"], "bf16"))
        assert len(w["layers"]) == cfg.layers
        for ly in w["layers"]:
            for key, _, dt in _LAYER:
                assert tuple(np.shape(ly[key])) == sh[key], key
                f.write(_raw(ly[key], dt))
        f.write(_raw(w["lnf"], "<f4"))
        f.write(_raw(w["lm_head"], "bf16"))


def read_config(path) -> GptOssConfig:
    h = Path(path).open("rb").read(128)
    v = struct.unpack("<13I4f4I4I7I", h)
    if v[0] != MAGIC:
        raise ValueError("not a gpt-oss weight file")
    return GptOssConfig(layers=v[1], hidden=v[2], inter=v[3], experts=v[4], top_k=v[5], n_q=v[6], n_kv=v[7], head_dim=v[8],
                        vocab=v[9], window=v[10], max_seq=v[11], batch=v[12], rope_theta=v[13], eps=v[14], alpha=v[15],
                        limit=v[16], seed=v[17], flags=v[18])


def load_checkpoint(model: GptOss, path) -> None:
    """Stream a weight file into a loaded instance, tensor by tensor (stage `setTensor`).  The instance's widths must
    be the file's; batch, max_seq, flags and the expert-parallel rank are the instance's own (an expert-parallel rank
    takes its slice of every expert tensor)."""
    c, fc = model.cfg, read_config(path)
    for k in ("layers", "hidden", "inter", "experts", "top_k", "n_q", "n_kv", "vocab"):
        if getattr(c, k) != getattr(fc, k):
            raise ValueError(f"weight file has {k} = {getattr(fc, k)}, the instance {getattr(c, k)}")
    sh = _shapes(c)
    data = np.memmap(path, dtype=np.uint8, mode="r")
    world = max(c.ep_world, 1) if c.flags & 128 else 1
    n_e = c.experts // world
    lo = c.ep_rank * n_e if world > 1 else 0
    off = 128

    def take(key, dt):
        nonlocal off
        n = int(np.prod(sh[key])) * (2 if dt == "bf16" else np.dtype(dt).itemsize)
        a = data[off:off + n]
        off += n
        return a

    def send(layer, kind, payload: bytes):
        model.base.execute(model.art.extras["setTensor"], struct.pack("<2I", layer, KIND[kind]) + payload)

    send(GLOBAL_LAYER, "embed", take("embed", "bf16").tobytes())
    for l in range(c.layers):
        t = {key: take(key, dt) for key, _, dt in _LAYER}
        for key, kind, dt in _LAYER:
            if key in ("gu_scales", "dn_scales"):
                continue
            if key in ("gu_codes", "dn_codes"):
                sk = key.replace("codes", "scales")
                codes = t[key].reshape(sh[key])[lo:lo + n_e]
                scales = t[sk].reshape(sh[sk])[lo:lo + n_e]
                send(l, kind, codes.tobytes() + scales.tobytes())
            else:
                send(l, kind, t[key].tobytes())
    send(GLOBAL_LAYER, "lnf", take("lnf", "<f4").tobytes())
    send(GLOBAL_LAYER, "lm_head", take("lm_head", "bf16").tobytes())
    if off != data.size:
        raise ValueError("weight file is longer than its header says")


def from_hf_state_dict(sd: dict, cfg: GptOssConfig) -> dict:
    """Hugging Face gpt-oss tensor names -> the weights dict of `write_checkpoint`.  `sd` maps names to NumPy arrays
    (MXFP4 expert tensors as stored in the checkpoint: `*_blocks` u8 [E, R, K/32, 16], `*_scales` u8 [E, R, K/32];
    everything else as float).  Not covered: the YaRN RoPE scaling of the released checkpoints (the stage program's
    RoPE table is the plain one)."""
    def g(name):
        return np.asarray(sd[name])
    w = {"embed": g("model.embed_tokens.weight").astype(np.float32), "lnf": g("model.norm.weight").astype(np.float32),
         "lm_head": g("lm_head.weight").astype(np.float32), "layers": []}
    for l in range(cfg.layers):
        p = f"model.layers.{l}."
        a, m = p + "self_attn.", p + "mlp."
        gu_b, dn_b = g(m + "experts.gate_up_proj_blocks"), g(m + "experts.down_proj_blocks")
        w["layers"].append({
            "ln1": g(p + "input_layernorm.weight").astype(np.float32),
            "wqkv": np.concatenate([g(a + f"{x}_proj.weight") for x in "qkv"], axis=0).astype(np.float32),
            "bqkv": np.concatenate([g(a + f"{x}_proj.bias") for x in "qkv"], axis=0).astype(np.float32),
            "sinks": g(a + "sinks").astype(np.float32),
            "wo": g(a + "o_proj.weight").astype(np.float32), "bo": g(a + "o_proj.bias").astype(np.float32),
            "ln2": g(p + "post_attention_layernorm.weight").astype(np.float32),
            "Wr": g(m + "router.weight").astype(np.float32), "br": g(m + "router.bias").astype(np.float32),
            "gu_codes": gu_b.reshape(*gu_b.shape[:2], -1), "gu_scales": g(m + "experts.gate_up_proj_scales"),
            "gu_bias": g(m + "experts.gate_up_proj_bias").astype(np.float32),
            "dn_codes": dn_b.reshape(*dn_b.shape[:2], -1), "dn_scales": g(m + "experts.down_proj_scales"),
            "dn_bias": g(m + "experts.down_proj_bias").astype(np.float32)})
    return w


# ---- Qwen2: the reference's flat f32 weight file -------------------------------------------------------------------
# tools/qwen2_convert.py:12-28, 101-141: f32 little endian, no header, in this order: embed_tokens [vocab][hidden]; per
# layer rms_attn [hidden], q_proj weight [n_q*64][hidden] and bias, k_proj weight [n_kv*64][hidden] and bias, v_proj
# weight and bias, o_proj weight [hidden][n_q*64], rms_ffn [hidden], gate_proj [inter][hidden], up_proj [inter][hidden],
# down_proj [hidden][inter]; then rms_final [hidden] and lm_head [vocab][hidden] (a copy of embed_tokens for the 0.5B
# model, which ties them).

def qwen2_flat_layout(cfg):
    """[(name, layer or None, shape)] in file order for a base_b200.qwen2.Qwen2Config."""
    H, F, QD, KVD, V = cfg.hidden, cfg.inter, cfg.n_q * cfg.head_dim, cfg.n_kv * cfg.head_dim, cfg.vocab
    out = [("embed", None, (V, H))]
    for l in range(cfg.layers):
        out += [("ln1", l, (H,)), ("wq", l, (QD, H)), ("bq", l, (QD,)), ("wk", l, (KVD, H)), ("bk", l, (KVD,)),
                ("wv", l, (KVD, H)), ("bv", l, (KVD,)), ("wo", l, (H, QD)), ("ln2", l, (H,)), ("wgate", l, (F, H)),
                ("wup", l, (F, H)), ("wdn", l, (H, F))]
    out += [("lnf", None, (H,)), ("lm_head", None, (V, H))]
    return out


def qwen2_flat_bytes(cfg) -> int:
    return 4 * sum(int(np.prod(shape)) for _, _, shape in qwen2_flat_layout(cfg))


def write_qwen2_flat(path, cfg, tensors: dict) -> None:
    """tensors: {(name, layer or None): array} with the names of qwen2_flat_layout."""
    with open(path, "wb") as f:
        for name, layer, shape in qwen2_flat_layout(cfg):
            a = np.asarray(tensors[(name, layer)], dtype="<f4")
            if a.shape != shape:
                raise ValueError(f"{name} of layer {layer}: shape {a.shape}, expected {shape}")
            f.write(a.tobytes())


def read_qwen2_flat(path, cfg) -> dict:
    """The file as {(name, layer or None): read-only array view} (memory-mapped)."""
    import os
    need = qwen2_flat_bytes(cfg)
    if os.path.getsize(path) != need:
        raise ValueError(f"{path}: {os.path.getsize(path)} bytes, the configuration needs {need}")
    mm = np.memmap(path, dtype="<f4", mode="r")
    out, at = {}, 0
    for name, layer, shape in qwen2_flat_layout(cfg):
        n = int(np.prod(shape))
        out[(name, layer)] = mm[at:at + n].reshape(shape)
        at += n
    return out


def qwen2_stage_tensors(cfg, flat: dict):
    """The stage program's tensors from the file's: yields (layer, kind, array) with wqkv = [q; k; v] rows and
    wgu = [gate; up] rows (layer 1000 = globals).  The stage ties lm_head to the embedding, as Qwen2-0.5B does: a
    file whose lm_head differs from its embedding is refused."""
    if not np.array_equal(flat[("embed", None)], flat[("lm_head", None)]):
        raise ValueError("lm_head differs from embed_tokens: the qwen2 stage program ties them")
    yield 1000, "embed", flat[("embed", None)]
    yield 1000, "lnf", flat[("lnf", None)]
    for l in range(cfg.layers):
        yield l, "ln1", flat[("ln1", l)]
        yield l, "wqkv", np.concatenate([flat[("wq", l)], flat[("wk", l)], flat[("wv", l)]], axis=0)
        yield l, "bqkv", np.concatenate([flat[("bq", l)], flat[("bk", l)], flat[("bv", l)]], axis=0)
        yield l, "wo", flat[("wo", l)]
        yield l, "ln2", flat[("ln2", l)]
        yield l, "wgu", np.concatenate([flat[("wgate", l)], flat[("wup", l)]], axis=0)
        yield l, "wdn", flat[("wdn", l)]


def load_qwen2_flat(model, path) -> None:
    """Replace the seeded weights of a base_b200.qwen2.Qwen2 instance by those of a flat weight file."""
    for layer, kind, a in qwen2_stage_tensors(model.cfg, read_qwen2_flat(path, model.cfg)):
        model.set_tensor(layer, kind, a)


def qwen2_flat_from_hf_state_dict(sd: dict, cfg) -> dict:
    """Hugging Face Qwen2 parameter names -> the file's tensors (tools/qwen2_convert.py:113-137)."""
    g = lambda k: np.asarray(sd[k], dtype=np.float32)
    out = {("embed", None): g("model.embed_tokens.weight"), ("lnf", None): g("model.norm.weight")}
    out[("lm_head", None)] = g("lm_head.weight") if "lm_head.weight" in sd else out[("embed", None)]
    for l in range(cfg.layers):
        p = f"model.layers.{l}"
        out.update({("ln1", l): g(f"{p}.input_layernorm.weight"), ("wq", l): g(f"{p}.self_attn.q_proj.weight"),
                    ("bq", l): g(f"{p}.self_attn.q_proj.bias"), ("wk", l): g(f"{p}.self_attn.k_proj.weight"),
                    ("bk", l): g(f"{p}.self_attn.k_proj.bias"), ("wv", l): g(f"{p}.self_attn.v_proj.weight"),
                    ("bv", l): g(f"{p}.self_attn.v_proj.bias"), ("wo", l): g(f"{p}.self_attn.o_proj.weight"),
                    ("ln2", l): g(f"{p}.post_attention_layernorm.weight"), ("wgate", l): g(f"{p}.mlp.gate_proj.weight"),
                    ("wup", l): g(f"{p}.mlp.up_proj.weight"), ("wdn", l): g(f"{p}.mlp.down_proj.weight")})
    return out
