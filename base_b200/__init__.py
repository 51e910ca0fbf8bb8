"""base_b200 — B200-native implementation of Base's quantized-inference hot path.

The product is the native library `libb200base.so` (C ABI in `include/`); this
package holds its sources (`csrc/`), the build step (`build.py`), a ctypes
binding (`lib()`), and `py_base`, a mirror of the reference's Python module of
that name (py-base/src/lib.rs:126-178) on top of the binding.

There is no CPU fallback: every compute entry point needs the library and a
CUDA device, and raises otherwise.
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path

_PKG = Path(__file__).resolve().parent
LIB_PATH = _PKG / "libb200base.so"
_lib = None


class NativeLibraryMissing(RuntimeError):
    pass


def lib() -> ctypes.CDLL:
    """The loaded native library with argument/return types declared."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        if os.environ.get("B200_NO_AUTOBUILD"):
            raise NativeLibraryMissing(f"{LIB_PATH} is not built; run `python -m base_b200.build`")
        from . import build as _build
        _build.build()
    L = ctypes.CDLL(str(LIB_PATH))
    c = ctypes
    vp, i32, i64, u32, u64 = c.c_void_p, c.c_int32, c.c_int64, c.c_uint32, c.c_uint64
    cp = c.c_char_p

    def sig(name, res, *args):
        f = getattr(L, name)
        f.restype = res
        f.argtypes = list(args)

    # --- b200abi.h
    sig("cl_cuda_init", None, c.POINTER(vp))
    sig("cl_cuda_cleanup", None, c.POINTER(vp))
    sig("cl_cuda_create_buffer", i32, vp, i64)
    sig("cl_cuda_free_buffer", i32, vp, i32)
    for n in ("cl_cuda_upload", "cl_cuda_upload_ptr", "cl_cuda_download", "cl_cuda_download_ptr"):
        sig(n, i32, vp, i32, vp, i64)
    sig("cl_cuda_upload_ptr_offset", i32, vp, i32, i64, vp, i64)
    sig("cl_cuda_download_ptr_offset", i32, vp, i32, i64, vp, i64)
    sig("cl_cuda_upload_ptr_async", i32, vp, i32, vp, i64, i32)
    sig("cl_cuda_upload_ptr_offset_async", i32, vp, i32, i64, vp, i64, i32)
    sig("cl_cuda_download_ptr_async", i32, vp, i32, vp, i64, i32)
    sig("cl_cuda_stream_create", i32, vp)
    sig("cl_cuda_stream_sync", i32, vp, i32)
    sig("cl_cuda_stream_destroy", i32, vp, i32)
    sig("cl_cuda_event_create", i32, vp)
    sig("cl_cuda_event_record", i32, vp, i32, i32)
    sig("cl_cuda_stream_wait_event", i32, vp, i32, i32)
    sig("cl_cuda_event_elapsed_ms_bits", i32, vp, i32, i32)
    sig("cl_cuda_event_destroy", i32, vp, i32)
    sig("cl_cuda_graph_begin_capture", i32, vp, i32)
    sig("cl_cuda_graph_end_capture", i32, vp, i32)
    sig("cl_cuda_graph_upload", i32, vp, i32, i32)
    sig("cl_cuda_graph_launch", i32, vp, i32, i32)
    sig("cl_cuda_graph_destroy", i32, vp, i32)
    sig("cl_cuda_pinned_alloc", i32, vp, i64)
    sig("cl_cuda_pinned_ptr", i64, vp, i32)
    sig("cl_cuda_pinned_free", i32, vp, i32)
    sig("cl_cuda_launch", i32, vp, vp, i32, vp, i32, i32, i32, i32, i32, i32)
    sig("cl_cuda_launch_named", i32, vp, vp, vp, i32, vp, i32, i32, i32, i32, i32, i32)
    sig("cl_cuda_launch_on_stream", i32, vp, vp, i32, vp, i32, i32, i32, i32, i32, i32, i32)
    sig("cl_cuda_launch_named_on_stream", i32, vp, vp, vp, i32, vp, i32, i32, i32, i32, i32, i32, i32)
    sig("cl_cuda_sync", i32, vp)
    sig("cl_cublas_sgemv", i32, vp, i32, i32, i32, i32, i32, i32, i32, i32)
    sig("cl_cublas_sgemv_on_stream", i32, vp, i32, i32, i32, i32, i32, i32, i32, i32, i32)
    sig("cl_cublas_sgemm", i32, vp, i32, i32, i32, i32, i32, i32, i32, i32, i32, i32)
    sig("cl_cublas_sgemm_strided_batched", i32, vp, i32, i32, i32, i32, i32, i32, i32, i64, i32, i64,
        i32, i32, i64, i32)
    sig("cl_cublas_sgemm_strided_batched_on_stream", i32, vp, i32, i32, i32, i32, i32, i32, i32, i64,
        i32, i64, i32, i32, i64, i32, i32)
    sig("cl_b200_load_module", i32, vp, vp, i64)
    sig("cl_b200_builtin_module", i32, vp)
    sig("cl_b200_launch", i32, vp, i32, cp, i32, vp, vp, i32, i32, i32, i32, i32, i32, i32, i32, i32, i32)
    sig("cl_b200_buffer_ptr", i64, vp, i32)
    sig("cl_b200_buffer_size", i64, vp, i32)
    sig("cl_b200_memset_async", i32, vp, i32, i64, i32, i64, i32)
    sig("cl_b200_copy_async", i32, vp, i32, i64, i32, i64, i64, i32)
    sig("cl_b200_device_ordinal", i32, vp)
    sig("cl_b200_copy_to_device_ptr", i32, vp, i32, i64, ctypes.c_uint64, i64, i32)
    sig("cl_b200_sm_count", i32, vp)
    sig("cl_b200_mem_free", i64, vp)
    sig("cl_b200_stream_handle", i64, vp, i32)
    sig("cl_b200_comm_unique_id", i32, vp)
    sig("cl_b200_comm_init", i32, vp, vp, i32, i32)
    sig("cl_b200_comm_world", i32, vp)
    sig("cl_b200_comm_all_gather", i32, vp, i32, i64, i32, i64, i32)
    sig("cl_b200_comm_all_to_all", i32, vp, i32, i32, i64, i32)
    sig("cl_b200_ipc_export", i32, vp, i32, vp)
    sig("cl_b200_ipc_open", i64, vp, vp)
    sig("cl_b200_ipc_close", i32, vp, i64)
    sig("cl_b200_last_error", cp)
    sig("cl_b200_argmax_noalloc", i32, vp, i32, i32, i32, vp, vp)
    sig("cl_b200_argmax_noalloc_error", cp)
    # --- b200base.h
    sig("b200_base_new", vp, cp, u64, c.POINTER(u64), vp, u64, c.POINTER(i32))
    sig("b200_base_free", None, vp)
    sig("b200_base_execute_into", i32, vp, u32, vp, u64, vp, u64)
    sig("b200_base_memory", vp, vp, c.POINTER(u64))
    sig("b200_base_fn_count", u32, vp)
    sig("b200_last_error", cp)
    sig("b200_artifact_from_json", vp, cp, u64)
    sig("b200_artifact_from_bytes", vp, vp, u64)
    sig("b200_artifact_free", None, vp)
    sig("b200_artifact_cranelift_ir", cp, vp)
    sig("b200_artifact_memory_size", u64, vp)
    sig("b200_artifact_io_offsets", None, vp, c.POINTER(u64))
    sig("b200_artifact_initial_memory", vp, vp, c.POINTER(u64))
    sig("b200_artifact_main_fn", u32, vp)
    sig("b200_artifact_extras_count", u32, vp)
    sig("b200_artifact_extra_name", cp, vp, u32)
    sig("b200_artifact_extra_fn", u32, vp, u32)
    sig("b200_base_from_artifact", vp, vp, c.POINTER(i32))
    sig("b200_plugin_count", u32)
    sig("b200_plugin_name", cp, u32)
    sig("b200_plugin_fn_count", u32, cp)
    sig("b200_plugin_fn_name", cp, cp, u32)
    _lib = L
    return L
