"""The allocation-free argmax entry point against the regular one.

Some users of this library cannot allocate device memory at the point where
they need the greedy token: they run inside a fixed pool, or in a serving
loop where cudaMalloc's device-wide synchronisation is not acceptable.  For
them `cl_b200_argmax_noalloc` keeps its scratch in a static array of the
library image.  This test drives it through the C-ABI with device pointers
and checks it against the regular `argmax_first` launch (scratch in buffers
the caller allocated), twice in a row, because the static scratch keeps what
the previous call left in it.  Collected last on purpose."""
import ctypes
import struct

import numpy as np
import pytest

from base_b200 import lib

pytestmark = pytest.mark.gpu

PARTS = 128


def regular_argmax(L, c, mod, logits_buf, out_buf, V, B, stride):
    pv = L.cl_cuda_create_buffer(c, B * PARTS * 4)
    pi = L.cl_cuda_create_buffer(c, B * PARTS * 4)
    tk = L.cl_cuda_create_buffer(c, B * 4)
    bind = struct.pack("<7i", logits_buf, out_buf, -1, -1, pv, pi, tk)
    args = struct.pack("<4i", V, B, stride, PARTS)
    assert L.cl_b200_launch(c, mod, b"argmax_first", 7, bind, args, len(args), PARTS, B, 1, 256, 1, 1, 0, -1, 0) == 0
    assert L.cl_cuda_sync(c) == 0
    out = np.zeros(B, dtype=np.int32)
    assert L.cl_cuda_download_ptr(c, out_buf, out.ctypes.data_as(ctypes.c_void_p), out.nbytes) == 0
    for b in (pv, pi, tk):
        L.cl_cuda_free_buffer(c, b)
    return out


def test_noalloc_argmax_matches_regular_entry_point_twice():
    L = lib()
    slot = ctypes.c_void_p(0)
    L.cl_cuda_init(ctypes.byref(slot))
    assert slot.value, L.cl_b200_last_error().decode()
    c = slot
    mod = L.cl_b200_builtin_module(c)
    assert mod >= 0
    rng = np.random.default_rng(77)
    for call, (V, B) in enumerate(((201088, 3), (50000, 5))):
        stride = V + 8
        logits = rng.standard_normal((B, stride)).astype(np.float32)
        logits[0, 123] = logits[0, 4567] = 9.5            # a tie: the smaller index must win
        lb = L.cl_cuda_create_buffer(c, logits.nbytes)
        o1 = L.cl_cuda_create_buffer(c, B * 4)
        o2 = L.cl_cuda_create_buffer(c, B * 4)
        assert L.cl_cuda_upload_ptr(c, lb, logits.ctypes.data_as(ctypes.c_void_p), logits.nbytes) == 0
        want = regular_argmax(L, c, mod, lb, o1, V, B, stride)
        np.testing.assert_array_equal(want, np.argmax(logits[:, :V], axis=1))
        rc = L.cl_b200_argmax_noalloc(ctypes.c_void_p(L.cl_b200_buffer_ptr(c, lb)), V, B, stride,
                                      ctypes.c_void_p(L.cl_b200_buffer_ptr(c, o2)), None)
        assert rc == 0, L.cl_b200_argmax_noalloc_error().decode()
        assert L.cl_cuda_sync(c) == 0
        got = np.zeros(B, dtype=np.int32)
        assert L.cl_cuda_download_ptr(c, o2, got.ctypes.data_as(ctypes.c_void_p), got.nbytes) == 0
        np.testing.assert_array_equal(got, want, err_msg=f"call {call}")
        assert got[0] == 123
    # beyond the built-in scratch: refused, nothing launched
    assert L.cl_b200_argmax_noalloc(ctypes.c_void_p(L.cl_b200_buffer_ptr(c, lb)), 100, 65, 100,
                                    ctypes.c_void_p(L.cl_b200_buffer_ptr(c, o2)), None) == -1
    assert b"exceed" in L.cl_b200_argmax_noalloc_error()
    L.cl_cuda_cleanup(ctypes.byref(slot))


def test_noalloc_argmax_is_ordered_after_a_kernel_on_the_library_stream():
    """The logits come from a kernel of this library on its main stream (a non-blocking stream, which the
    default stream does not wait for); the argmax is given that stream's handle and nothing synchronises in
    between, on two calls in a row.  A serving loop that may not allocate uses it exactly like this."""
    L = lib()
    slot = ctypes.c_void_p(0)
    L.cl_cuda_init(ctypes.byref(slot))
    assert slot.value, L.cl_b200_last_error().decode()
    c = slot
    mod = L.cl_b200_builtin_module(c)
    handle = L.cl_b200_stream_handle(c, -1)
    assert handle != 0 and L.cl_b200_stream_handle(c, 99) == 0
    from oracle import synth
    V, B = 150000, 4
    lb = L.cl_cuda_create_buffer(c, B * V * 4)
    ob = L.cl_cuda_create_buffer(c, B * 4)
    for call, seed in enumerate((3, 4)):
        # synth_fill, kind 2: f32 N(0, 1) values from (seed, tensor 77, index), generated on the main stream
        args = struct.pack("<Q2Iif2iQ", B * V, 77, seed, 2, 1.0 / 209.0232, 0, 1, 0)
        bind = struct.pack("<i", lb)
        assert L.cl_b200_launch(c, mod, b"synth_fill", 1, bind, args, len(args), 148 * 8, 1, 1, 256, 1, 1, 0, -1, 0) == 0
        rc = L.cl_b200_argmax_noalloc(ctypes.c_void_p(L.cl_b200_buffer_ptr(c, lb)), V, B, V,
                                      ctypes.c_void_p(L.cl_b200_buffer_ptr(c, ob)), ctypes.c_void_p(handle))
        assert rc == 0, L.cl_b200_argmax_noalloc_error().decode()
        assert L.cl_cuda_sync(c) == 0
        got = np.zeros(B, dtype=np.int32)
        assert L.cl_cuda_download_ptr(c, ob, got.ctypes.data_as(ctypes.c_void_p), got.nbytes) == 0
        want = np.argmax(synth.normal(B * V, 77, seed, 1.0).reshape(B, V), axis=1)
        np.testing.assert_array_equal(got, want, err_msg=f"call {call}")
    L.cl_cuda_cleanup(ctypes.byref(slot))
