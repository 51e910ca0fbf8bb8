"""MXFP4 GEMV on the block-scaled tensor cores (tcgen05.mma.kind::mxf4.block_scale):
E2M1 codes and UE8M0 scales go to the tensor core as stored; the f32 activation
vector is expanded into E2M1 terms.  Checked against the NumPy dequantise-and-multiply."""
import ctypes
import struct

import numpy as np
import pytest

from base_b200 import lib
from oracle import moe_oracle

# a kernel that never returns must end the test process, not hold the GPU
pytestmark = [pytest.mark.gpu, pytest.mark.timeout(120, method="thread")]


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


def run_gemv(L, c, codes, scales, x, terms):
    rows, K = codes.shape[0], codes.shape[1] * 2
    kblocks, atoms = K // 32, (K // 32 + 3) // 4
    m = load_probe_module(L, c)
    ins = [np.ascontiguousarray(codes), np.ascontiguousarray(scales), np.ascontiguousarray(x, dtype=np.float32)]
    bufs = [L.cl_cuda_create_buffer(c, a.nbytes) for a in ins] + [L.cl_cuda_create_buffer(c, rows * 4),
                                                                   L.cl_cuda_create_buffer(c, 4)]
    assert min(bufs) >= 0
    for buf, arr in zip(bufs, ins):
        assert L.cl_cuda_upload_ptr(c, buf, arr.ctypes.data_as(ctypes.c_void_p), arr.nbytes) == 0
    smem = kblocks * 256 + 2048 + atoms * 512 + (kblocks + 1) * 512 + atoms * 512
    bind = struct.pack("<5i", *bufs)
    args = struct.pack("<2i", K, terms)
    rc = L.cl_b200_launch(c, m, b"mxf4_tc_gemv_test", 5, bind, args, len(args), rows // 32, 1, 1, 128, 1, 1, smem, -1, 0)
    assert rc == 0, L.cl_b200_last_error().decode()
    assert L.cl_cuda_sync(c) == 0, L.cl_b200_last_error().decode()
    st = np.zeros(1, np.int32)
    assert L.cl_cuda_download_ptr(c, bufs[4], st.ctypes.data_as(ctypes.c_void_p), 4) == 0
    assert st[0] == 0, f"kernel gave up waiting (code {st[0]})"
    y = np.zeros(rows, np.float32)
    assert L.cl_cuda_download_ptr(c, bufs[3], y.ctypes.data_as(ctypes.c_void_p), y.nbytes) == 0
    return y


def check(L, c, rows, K, terms, tol):
    rng = np.random.default_rng(rows * 7 + K + terms)
    codes = rng.integers(0, 256, size=(rows, K // 2), dtype=np.uint8)
    scales = rng.integers(117, 124, size=(rows, K // 32), dtype=np.uint8)
    x = rng.standard_normal(K).astype(np.float32)
    y = run_gemv(L, c, codes, scales, x, terms)
    W = moe_oracle.mx_dequant(codes, scales).astype(np.float64)
    ref = W @ x.astype(np.float64)
    err = np.abs(y - ref).max() / np.abs(ref).max()
    assert err <= tol, f"max error {err:.3e} of max |y|"


@pytest.mark.parametrize("rows,K,terms,tol", [(32, 64, 12, 1e-5), (64, 512, 12, 1e-5), (96, 2880, 12, 1e-5),
                                               (32, 2880, 6, 2e-3), (32, 1024, 16, 2e-6)])
def test_block_scaled_mxfp4_gemv_matches_dequantised_product(ctx, rows, K, terms, tol):
    L, c = ctx
    check(L, c, rows, K, terms, tol)


def test_issue_rate_probe_runs(ctx):
    """The rate probe (bench material) completes and reports a positive cycle count per CTA."""
    L, c = ctx
    m = load_probe_module(L, c)
    bufs = [L.cl_cuda_create_buffer(c, 8 * 4), L.cl_cuda_create_buffer(c, 4)]
    bind = struct.pack("<2i", *bufs)
    args = struct.pack("<8i", 32, 64, 2, 0, 0, 0, 0, 7)
    rc = L.cl_b200_launch(c, m, b"mxf4_tc_rate_probe", 2, bind, args, len(args), 4, 1, 1, 128, 1, 1, 4608 + 32 * 32 + 4096, -1, 0)
    assert rc == 0, L.cl_b200_last_error().decode()
    assert L.cl_cuda_sync(c) == 0, L.cl_b200_last_error().decode()
    cyc = np.zeros(4, np.int64)
    assert L.cl_cuda_download_ptr(c, bufs[0], cyc.ctypes.data_as(ctypes.c_void_p), cyc.nbytes) == 0
    assert (cyc > 0).all()
