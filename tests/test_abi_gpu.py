"""C-ABI conformance on a real device, following the reference's unit tests in
base/src/ffi/cuda.rs:1993-2891 (ids, -1 conventions, round trips, launches,
streams, events, graphs, pinned memory, the cuBLAS-shaped calls)."""
import ctypes
import struct

import numpy as np
import pytest

from base_b200 import lib

pytestmark = pytest.mark.gpu

VEC_ADD_PTX = b"""
.version 7.5
.target sm_75
.address_size 64
.visible .entry main(.param .u64 b0_ptr, .param .u64 b1_ptr, .param .u64 b2_ptr)
{
  .reg .b32 %r<6>;
  .reg .b64 %rd<10>;
  .reg .f32 %f<4>;
  ld.param.u64 %rd1, [b0_ptr];
  ld.param.u64 %rd2, [b1_ptr];
  ld.param.u64 %rd3, [b2_ptr];
  cvta.to.global.u64 %rd1, %rd1;
  cvta.to.global.u64 %rd2, %rd2;
  cvta.to.global.u64 %rd3, %rd3;
  mov.u32 %r1, %tid.x;
  mov.u32 %r2, %ctaid.x;
  mov.u32 %r3, %ntid.x;
  mad.lo.s32 %r4, %r2, %r3, %r1;
  mul.wide.s32 %rd4, %r4, 4;
  add.s64 %rd5, %rd1, %rd4;
  add.s64 %rd6, %rd2, %rd4;
  add.s64 %rd7, %rd3, %rd4;
  ld.global.f32 %f1, [%rd5];
  ld.global.f32 %f2, [%rd6];
  add.rn.f32 %f3, %f1, %f2;
  st.global.f32 [%rd7], %f3;
  ret;
}
.visible .entry scale2(.param .u64 b0_ptr)
{
  .reg .b32 %r<6>;
  .reg .b64 %rd<6>;
  .reg .f32 %f<3>;
  ld.param.u64 %rd1, [b0_ptr];
  cvta.to.global.u64 %rd1, %rd1;
  mov.u32 %r1, %tid.x;
  mov.u32 %r2, %ctaid.x;
  mov.u32 %r3, %ntid.x;
  mad.lo.s32 %r4, %r2, %r3, %r1;
  mul.wide.s32 %rd2, %r4, 4;
  add.s64 %rd3, %rd1, %rd2;
  ld.global.f32 %f1, [%rd3];
  add.rn.f32 %f2, %f1, %f1;
  st.global.f32 [%rd3], %f2;
  ret;
}
\0"""


@pytest.fixture()
def ctx():
    L = lib()
    slot = ctypes.c_void_p(0)
    L.cl_cuda_init(ctypes.byref(slot))
    assert slot.value, "no GPU? " + L.cl_b200_last_error().decode()
    yield L, slot
    L.cl_cuda_cleanup(ctypes.byref(slot))
    assert slot.value is None


def up(L, c, buf, arr):
    a = np.ascontiguousarray(arr)
    return L.cl_cuda_upload_ptr(c, buf, a.ctypes.data_as(ctypes.c_void_p), a.nbytes)


def down(L, c, buf, n, dtype=np.float32):
    out = np.zeros(n, dtype=dtype)
    assert L.cl_cuda_download_ptr(c, buf, out.ctypes.data_as(ctypes.c_void_p), out.nbytes) == 0
    return out


def f32bits(v):
    return struct.unpack("<i", struct.pack("<f", v))[0]


def test_buffer_ids_sizes_and_round_trips(ctx):
    L, c = ctx
    assert [L.cl_cuda_create_buffer(c, 64) for _ in range(3)] == [0, 1, 2]   # cuda.rs:2191-2203
    assert L.cl_cuda_create_buffer(c, 0) == -1 and L.cl_cuda_create_buffer(c, -5) == -1
    assert np.all(down(L, c, 0, 16) == 0)                                     # zero-filled
    src = np.arange(16, dtype=np.float32)
    assert up(L, c, 0, src) == 0
    np.testing.assert_array_equal(down(L, c, 0, 16), src)
    big = np.zeros(17, dtype=np.float32)
    assert up(L, c, 0, big) == -1                                             # too large
    assert L.cl_cuda_upload_ptr(c, 7, src.ctypes.data_as(ctypes.c_void_p), 4) == -1   # bad id
    # offset forms, cuda.rs:2249-2276
    part = np.array([100, 101], dtype=np.float32)
    assert L.cl_cuda_upload_ptr_offset(c, 0, 8, part.ctypes.data_as(ctypes.c_void_p), 8) == 0
    got = np.zeros(2, dtype=np.float32)
    assert L.cl_cuda_download_ptr_offset(c, 0, 8, got.ctypes.data_as(ctypes.c_void_p), 8) == 0
    np.testing.assert_array_equal(got, part)
    assert L.cl_cuda_upload_ptr_offset(c, 0, 60, part.ctypes.data_as(ctypes.c_void_p), 8) == -1
    assert L.cl_cuda_download_ptr_offset(c, 0, -4, got.ctypes.data_as(ctypes.c_void_p), 8) == -1
    assert L.cl_cuda_free_buffer(c, 1) == 0 and L.cl_cuda_free_buffer(c, 1) == -1   # double free
    assert L.cl_cuda_create_buffer(c, 8) == 3                                 # ids are not reused
    assert L.cl_b200_buffer_size(c, 0) == 64 and L.cl_b200_buffer_ptr(c, 0) != 0
    assert L.cl_b200_buffer_ptr(c, 1) == 0


def test_ptx_launch_cache_named_and_argument_checks(ctx):
    L, c = ctx
    n = 256
    a, b = np.arange(n, dtype=np.float32), np.full(n, 0.5, dtype=np.float32)
    ids = [L.cl_cuda_create_buffer(c, n * 4) for _ in range(3)]
    up(L, c, ids[0], a), up(L, c, ids[1], b)
    text = ctypes.create_string_buffer(VEC_ADD_PTX)
    bind = struct.pack("<3i", *ids)
    for _ in range(2):                                   # second launch hits the module cache
        assert L.cl_cuda_launch(c, text, 3, bind, n // 64, 1, 1, 64, 1, 1) == 0
    assert L.cl_cuda_sync(c) == 0
    np.testing.assert_array_equal(down(L, c, ids[2], n), a + b)
    assert L.cl_cuda_launch_named(c, text, b"scale2", 1, struct.pack("<i", ids[2]), n // 64, 1, 1, 64, 1, 1) == 0
    assert L.cl_cuda_sync(c) == 0
    np.testing.assert_array_equal(down(L, c, ids[2], n), 2 * (a + b))
    assert L.cl_cuda_launch(c, text, 3, bind, 0, 1, 1, 64, 1, 1) == -1       # bad grid
    assert L.cl_cuda_launch(c, text, 3, bind, 1, 1, 1, 64, 0, 1) == -1       # bad block
    assert L.cl_cuda_launch(c, text, -1, bind, 1, 1, 1, 64, 1, 1) == -1      # bad n_bufs
    assert L.cl_cuda_launch(c, text, 3, struct.pack("<3i", ids[0], 99, ids[2]), 1, 1, 1, 64, 1, 1) == -1
    assert L.cl_cuda_launch_named(c, text, b"nope", 1, struct.pack("<i", ids[2]), 1, 1, 1, 64, 1, 1) == -1


def test_streams_events_graphs_pinned(ctx):
    L, c = ctx
    n = 1024
    buf = L.cl_cuda_create_buffer(c, n * 4)
    s0 = L.cl_cuda_stream_create(c)
    s1 = L.cl_cuda_stream_create(c)
    assert (s0, s1) == (0, 1)
    e0, e1 = L.cl_cuda_event_create(c), L.cl_cuda_event_create(c)
    assert L.cl_cuda_event_elapsed_ms_bits(c, e0, e1) == -1                   # unrecorded
    pid = L.cl_cuda_pinned_alloc(c, n * 4)
    assert pid == 0 and L.cl_cuda_pinned_alloc(c, 0) == -1
    hp = L.cl_cuda_pinned_ptr(c, pid)
    host = np.ctypeslib.as_array((ctypes.c_float * n).from_address(hp))
    host[:] = np.arange(n, dtype=np.float32)
    text = ctypes.create_string_buffer(VEC_ADD_PTX)
    assert L.cl_cuda_event_record(c, e0, s0) == 0
    assert L.cl_cuda_upload_ptr_async(c, buf, hp, n * 4, s0) == 0
    assert L.cl_cuda_launch_named_on_stream(c, text, b"scale2", 1, struct.pack("<i", buf), n // 128, 1, 1, 128, 1, 1, s0) == 0
    assert L.cl_cuda_event_record(c, e1, s0) == 0
    # s1 waits for e1 before reading back
    assert L.cl_cuda_stream_wait_event(c, s1, e1) == 0
    host2_id = L.cl_cuda_pinned_alloc(c, n * 4)
    hp2 = L.cl_cuda_pinned_ptr(c, host2_id)
    assert L.cl_cuda_download_ptr_async(c, buf, hp2, n * 4, s1) == 0
    assert L.cl_cuda_stream_sync(c, s1) == 0
    got = np.ctypeslib.as_array((ctypes.c_float * n).from_address(hp2))
    np.testing.assert_array_equal(got, 2 * np.arange(n, dtype=np.float32))
    bits = L.cl_cuda_event_elapsed_ms_bits(c, e0, e1)
    ms = struct.unpack("<f", struct.pack("<i", bits))[0]
    assert bits != -1 and 0.0 <= ms < 1000.0
    # graph: capture two doublings, replay twice -> x16 overall
    assert L.cl_cuda_graph_begin_capture(c, s0) == 0
    for _ in range(2):
        assert L.cl_cuda_launch_named_on_stream(c, text, b"scale2", 1, struct.pack("<i", buf), n // 128, 1, 1, 128, 1, 1, s0) == 0
    g = L.cl_cuda_graph_end_capture(c, s0)
    assert g == 0
    assert L.cl_cuda_graph_upload(c, g, s0) == 0
    assert L.cl_cuda_graph_launch(c, g, s0) == 0 and L.cl_cuda_graph_launch(c, g, s0) == 0
    assert L.cl_cuda_stream_sync(c, s0) == 0
    np.testing.assert_array_equal(down(L, c, buf, n), 32 * np.arange(n, dtype=np.float32))
    assert L.cl_cuda_graph_launch(c, 5, s0) == -1
    assert L.cl_cuda_graph_destroy(c, g) == 0 and L.cl_cuda_graph_destroy(c, g) == -1
    assert L.cl_cuda_event_destroy(c, e0) == 0 and L.cl_cuda_event_destroy(c, e0) == -1
    assert L.cl_cuda_stream_destroy(c, s1) == 0 and L.cl_cuda_stream_sync(c, s1) == -1
    assert L.cl_cuda_pinned_free(c, pid) == 0 and L.cl_cuda_pinned_free(c, pid) == -1
    assert L.cl_cuda_pinned_ptr(c, pid) == 0


def test_sgemv_sgemm_reference_cases(ctx):
    L, c = ctx
    # cuda.rs:2706-2760 style: column-major 2x3 A, both transposes
    A = np.array([1, 2, 3, 4, 5, 6], dtype=np.float32)      # col-major m=2,n=3: [[1,3,5],[2,4,6]]
    a = L.cl_cuda_create_buffer(c, 24)
    x3 = L.cl_cuda_create_buffer(c, 12)
    y2 = L.cl_cuda_create_buffer(c, 8)
    up(L, c, a, A), up(L, c, x3, np.array([1, 1, 1], dtype=np.float32))
    assert L.cl_cublas_sgemv(c, 0, 2, 3, f32bits(1.0), a, x3, f32bits(0.0), y2) == 0
    assert L.cl_cuda_sync(c) == 0
    np.testing.assert_allclose(down(L, c, y2, 2), [9, 12])
    up(L, c, y2, np.array([1, 2], dtype=np.float32))
    y3 = L.cl_cuda_create_buffer(c, 12)
    up(L, c, y3, np.array([10, 10, 10], dtype=np.float32))
    assert L.cl_cublas_sgemv(c, 1, 2, 3, f32bits(2.0), a, y2, f32bits(0.5), y3) == 0
    assert L.cl_cuda_sync(c) == 0
    np.testing.assert_allclose(down(L, c, y3, 3), 2 * np.array([5, 11, 17]) + 5)
    assert L.cl_cublas_sgemv(c, 1, 0, 3, 0, a, y2, 0, y3) == -1
    assert L.cl_cublas_sgemv(c, 1, 2, 3, 0, 99, y2, 0, y3) == -1
    # realistic decode shape: row-major W[rows, cols] . x  == sgemv(T, m=cols, n=rows)
    r = np.random.default_rng(5)
    rows, cols = 4864, 896
    W = (r.standard_normal((rows, cols)) * 0.02).astype(np.float32)
    x = r.standard_normal(cols).astype(np.float32)
    wb, xb, yb = (L.cl_cuda_create_buffer(c, W.nbytes), L.cl_cuda_create_buffer(c, x.nbytes),
                  L.cl_cuda_create_buffer(c, rows * 4))
    up(L, c, wb, W), up(L, c, xb, x)
    assert L.cl_cublas_sgemv(c, 1, cols, rows, f32bits(1.0), wb, xb, f32bits(0.0), yb) == 0
    assert L.cl_cuda_sync(c) == 0
    ref = (W.astype(np.float64) @ x.astype(np.float64))
    got = down(L, c, yb, rows)
    assert np.abs(got - ref).max() / np.abs(ref).max() < 1e-5
    # strided batched, the attention-score shape of lean/lib/AlgorithmLib/Cuda.lean:313-332
    seq, nq, hd, nkv = 37, 7, 64, 2
    K = r.standard_normal((nkv, 64, hd)).astype(np.float32)        # [kv][MAX=64][hd]
    Q = r.standard_normal((nkv, nq, hd)).astype(np.float32)
    kb, qb = L.cl_cuda_create_buffer(c, K.nbytes), L.cl_cuda_create_buffer(c, Q.nbytes)
    sb = L.cl_cuda_create_buffer(c, nkv * nq * seq * 4)
    up(L, c, kb, K), up(L, c, qb, Q)
    assert L.cl_cublas_sgemm_strided_batched(c, 1, 0, seq, nq, hd, f32bits(0.125), kb, 64 * hd, qb, nq * hd,
                                             f32bits(0.0), sb, nq * seq, nkv) == 0
    assert L.cl_cuda_sync(c) == 0
    S = down(L, c, sb, nkv * nq * seq).reshape(nkv, nq, seq)
    ref = 0.125 * np.einsum("bsh,bqh->bqs", K[:, :seq].astype(np.float64), Q.astype(np.float64))
    assert np.abs(S - ref).max() < 1e-4
    c2 = L.cl_cuda_create_buffer(c, 2 * 2 * 4)
    a2 = L.cl_cuda_create_buffer(c, 2 * 3 * 4)
    b2 = L.cl_cuda_create_buffer(c, 3 * 2 * 4)
    up(L, c, a2, np.array([1, 2, 3, 4, 5, 6], dtype=np.float32))    # 2x3 col-major
    up(L, c, b2, np.array([1, 0, 1, 0, 1, 1], dtype=np.float32))    # 3x2 col-major
    assert L.cl_cublas_sgemm(c, 0, 0, 2, 2, 3, f32bits(1.0), a2, b2, f32bits(0.0), c2) == 0
    assert L.cl_cuda_sync(c) == 0
    np.testing.assert_allclose(down(L, c, c2, 4), [6, 8, 8, 10])


def test_builtin_module_and_b200_launch_checks(ctx):
    L, c = ctx
    m = L.cl_b200_builtin_module(c)
    assert m >= 0 and L.cl_b200_builtin_module(c) == m
    assert L.cl_b200_sm_count(c) > 0 and L.cl_b200_mem_free(c) > 0
    buf = L.cl_cuda_create_buffer(c, 64)
    bind = struct.pack("<i", buf)
    assert L.cl_b200_launch(c, m, b"no_such_kernel", 1, bind, None, 0, 1, 1, 1, 32, 1, 1, 0, -1, 0) == -1
    assert L.cl_b200_launch(c, m + 5, b"sgemv_t_f32", 1, bind, None, 0, 1, 1, 1, 32, 1, 1, 0, -1, 0) == -1
    assert L.cl_b200_launch(c, m, b"sgemv_t_f32", 1, bind, None, 0, 0, 1, 1, 32, 1, 1, 0, -1, 0) == -1
    assert L.cl_b200_memset_async(c, buf, 0, 0xAB, 64, -1) == 0
    assert L.cl_b200_memset_async(c, buf, 60, 0, 8, -1) == -1
    assert L.cl_cuda_sync(c) == 0
    assert np.all(down(L, c, buf, 64, np.uint8) == 0xAB)


@pytest.mark.parametrize("n,m", [(896, 4864), (2048, 4096), (8192, 2048), (16384, 2048)])
def test_committed_fold_gemv_is_bit_exact_on_the_reference_inputs(n, m):
    """The reference checks its proven GEMV kernels bit for bit against a CPU fold written in the committed order
    (applications/gemv-warp/src/main.rs:55-56, 129-148, 184-189: a[i] = ((i % 251) - 125) * 1e-3,
    x[i] = ((i % 97) - 48) * 1e-2, these four shapes).  `gemv_warp_fold_f32` commits to the same order; the oracle
    restates the reference's CPU image (applications/warp-check/src/lib.rs:28-116)."""
    import ctypes
    import struct
    from base_b200 import lib
    from oracle import c_oracle
    L = lib()
    slot = ctypes.c_void_p(0)
    L.cl_cuda_init(ctypes.byref(slot))
    assert slot.value
    c = slot
    i = np.arange(m * n, dtype=np.int64)
    a = (((i % 251).astype(np.float32) - np.float32(125.0)) * np.float32(0.001)).astype(np.float32).reshape(m, n)
    x = (((np.arange(n) % 97).astype(np.float32) - np.float32(48.0)) * np.float32(0.01)).astype(np.float32)
    mod = L.cl_b200_builtin_module(c)
    ba, bx, by = (L.cl_cuda_create_buffer(c, a.nbytes), L.cl_cuda_create_buffer(c, x.nbytes), L.cl_cuda_create_buffer(c, m * 4))
    assert L.cl_cuda_upload_ptr(c, ba, a.ctypes.data_as(ctypes.c_void_p), a.nbytes) == 0
    assert L.cl_cuda_upload_ptr(c, bx, x.ctypes.data_as(ctypes.c_void_p), x.nbytes) == 0
    for walk in (0, 1, 2):                                   # vec4, strided, blocked
        args = struct.pack("<3i", m, n, walk)
        assert L.cl_b200_launch(c, mod, b"gemv_warp_fold_f32", 3, struct.pack("<3i", ba, bx, by), args, len(args),
                                (m + 7) // 8, 1, 1, 256, 1, 1, 0, -1, 0) == 0
        assert L.cl_cuda_sync(c) == 0
        y = np.zeros(m, dtype=np.float32)
        assert L.cl_cuda_download_ptr(c, by, y.ctypes.data_as(ctypes.c_void_p), y.nbytes) == 0
        want = c_oracle.warp_fold_gemv(a, x, walk)
        np.testing.assert_array_equal(y.view(np.uint32), want.view(np.uint32), err_msg=f"walk {walk}")
    L.cl_cuda_cleanup(ctypes.byref(slot))
