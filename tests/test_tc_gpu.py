"""tcgen05 building blocks: the one-CTA bf16 GEMM (tensor memory accumulator,
shared-memory matrix descriptors, tcgen05.ld read-back) against NumPy.
Inputs are bf16-exact, so the f32 result must match to accumulation rounding."""
import ctypes
import struct

import numpy as np
import pytest

from base_b200 import lib
from oracle import synth

pytestmark = pytest.mark.gpu


def load_probe_module(L, c):
    """The test/probe kernels live in their own cubin (tests/kernels/probe_kernels.cu), not in the library's image."""
    from conftest import build_probe_kernels
    image = build_probe_kernels().read_bytes()
    buf = ctypes.create_string_buffer(image, len(image))
    m = L.cl_b200_load_module(c, ctypes.cast(buf, ctypes.c_void_p), len(image))
    assert m >= 0, L.cl_b200_last_error().decode()
    return m


@pytest.fixture()
def ctx():
    L = lib()
    slot = ctypes.c_void_p(0)
    L.cl_cuda_init(ctypes.byref(slot))
    assert slot.value, "no GPU? " + L.cl_b200_last_error().decode()
    yield L, slot
    L.cl_cuda_cleanup(ctypes.byref(slot))


def bf16_round(x):
    bits = synth.f32_to_bf16_bits(x.reshape(-1)).astype(np.uint32) << 16
    return bits.view(np.float32).reshape(x.shape), (bits >> 16).astype(np.uint16).reshape(x.shape)


@pytest.mark.parametrize("N,K", [(64, 64), (128, 256), (256, 2880 // 64 * 64), (16, 128)])
def test_one_cta_bf16_gemm_matches_numpy(ctx, N, K):
    L, c = ctx
    rng = np.random.default_rng(N + K)
    a32, a16 = bf16_round(rng.standard_normal((128, K)).astype(np.float32))
    b32, b16 = bf16_round(rng.standard_normal((N, K)).astype(np.float32))
    m = load_probe_module(L, c)
    bufs = [L.cl_cuda_create_buffer(c, a16.nbytes), L.cl_cuda_create_buffer(c, b16.nbytes),
            L.cl_cuda_create_buffer(c, 128 * N * 4), L.cl_cuda_create_buffer(c, 4)]
    assert min(bufs) >= 0
    for buf, arr in ((bufs[0], a16), (bufs[1], b16)):
        arr = np.ascontiguousarray(arr)
        assert L.cl_cuda_upload_ptr(c, buf, arr.ctypes.data_as(ctypes.c_void_p), arr.nbytes) == 0
    bind = struct.pack("<4i", *bufs)
    args = struct.pack("<2i", N, K)
    rc = L.cl_b200_launch(c, m, b"tc_gemm_test", 4, bind, args, len(args), 1, 1, 1, 128, 1, 1, 16384 + N * 128, -1, 0)
    assert rc == 0, L.cl_b200_last_error().decode()
    assert L.cl_cuda_sync(c) == 0, L.cl_b200_last_error().decode()
    st = np.zeros(1, np.int32)
    assert L.cl_cuda_download_ptr(c, bufs[3], st.ctypes.data_as(ctypes.c_void_p), 4) == 0
    assert st[0] == 0, f"kernel gave up waiting (code {st[0]})"
    out = np.zeros((128, N), np.float32)
    assert L.cl_cuda_download_ptr(c, bufs[2], out.ctypes.data_as(ctypes.c_void_p), out.nbytes) == 0
    ref = a32.astype(np.float64) @ b32.astype(np.float64).T
    assert np.abs(out - ref).max() <= 2e-5 * np.abs(ref).max() + 1e-6
