"""Host logic of the runtime and the C-ABI surface, without a GPU.  Modelled
on the reference's py-base/tests/test_base.py and the non-CUDA parts of
base/tests/integration.rs."""
import ctypes
import json
import re
import struct
from pathlib import Path

import pytest

from base_b200 import lib, py_base

ROOT = Path(__file__).resolve().parent.parent


def _declared_symbols():
    names = []
    for h in sorted((ROOT / "include").glob("*.h")):
        text = re.sub(r"/\*.*?\*/", "", h.read_text(), flags=re.S)
        names += re.findall(r"\b((?:cl_|b200_)[a-z0-9_]+)\s*\(", text)
    return sorted(set(names))


def test_library_exports_every_declared_symbol():
    L = ctypes.CDLL(str(ROOT / "base_b200" / "libb200base.so")) if (ROOT / "base_b200" / "libb200base.so").exists() else lib()
    syms = _declared_symbols()
    assert len(syms) > 60
    missing = [s for s in syms if not hasattr(L, s)]
    assert not missing, missing


def test_reference_ffi_names_are_all_present():
    # The 39 CUDA/cuBLAS symbols the reference registers (base/src/jit.rs:47-88).
    ref = """cl_cuda_init cl_cuda_create_buffer cl_cuda_upload cl_cuda_upload_ptr cl_cuda_upload_ptr_offset
    cl_cuda_upload_ptr_async cl_cuda_upload_ptr_offset_async cl_cuda_download cl_cuda_download_ptr
    cl_cuda_download_ptr_offset cl_cuda_download_ptr_async cl_cuda_free_buffer cl_cuda_stream_create
    cl_cuda_stream_sync cl_cuda_stream_destroy cl_cuda_event_create cl_cuda_event_record
    cl_cuda_stream_wait_event cl_cuda_event_elapsed_ms_bits cl_cuda_event_destroy
    cl_cuda_graph_begin_capture cl_cuda_graph_end_capture cl_cuda_graph_upload cl_cuda_graph_launch
    cl_cuda_graph_destroy cl_cuda_pinned_alloc cl_cuda_pinned_ptr cl_cuda_pinned_free cl_cuda_launch
    cl_cuda_launch_named cl_cuda_launch_on_stream cl_cuda_launch_named_on_stream cl_cuda_sync
    cl_cuda_cleanup cl_cublas_sgemm cl_cublas_sgemv cl_cublas_sgemv_on_stream
    cl_cublas_sgemm_strided_batched cl_cublas_sgemm_strided_batched_on_stream""".split()
    assert len(ref) == 39
    L = lib()
    for s in ref:
        assert hasattr(L, s), s


def test_null_context_returns_minus_one():
    # base/src/ffi/cuda.rs:2840-2884
    L = lib()
    assert L.cl_cuda_create_buffer(None, 16) == -1
    assert L.cl_cuda_free_buffer(None, 0) == -1
    assert L.cl_cuda_upload_ptr(None, 0, None, 0) == -1
    assert L.cl_cuda_sync(None) == -1
    assert L.cl_cuda_stream_create(None) == -1
    assert L.cl_cuda_event_create(None) == -1
    assert L.cl_cuda_pinned_alloc(None, 16) == -1
    assert L.cl_cuda_pinned_ptr(None, 0) == 0
    assert L.cl_cublas_sgemv(None, 1, 2, 2, 0, 0, 1, 0, 2) == -1
    assert L.cl_b200_launch(None, 0, b"k", 0, None, None, 0, 1, 1, 1, 1, 1, 1, 0, -1, 0) == -1
    slot = ctypes.c_void_p(0)
    L.cl_cuda_cleanup(ctypes.byref(slot))          # no-op on a null slot content
    L.cl_cuda_cleanup(None)
    assert slot.value is None


IO = py_base.IoOffsets(8, 16, 24, 32)   # the compact offsets of base/tests/integration.rs:11-18


def test_empty_ir_has_no_functions_and_execute_succeeds():
    # base/src/lib.rs:65-70; base/tests/integration.rs:2459-2469
    b = py_base.Base(py_base.Setup("", 0, IO))
    assert b.execute(py_base.Algorithm(0)) == []
    assert b.execute(py_base.Algorithm(12345)) == []


def test_memory_is_sized_like_the_reference():
    # max(memory_size, len(initial_memory), out_len offset + 8): base/src/lib.rs:36-46
    assert len(py_base.Base(py_base.Setup("", 0, IO)).memory()) == 40
    assert len(py_base.Base(py_base.Setup("", 4096, IO)).memory()) == 4096
    b = py_base.Base(py_base.Setup("", 16, IO, bytes(range(100))))
    m = b.memory()
    assert len(m) == 100 and bytes(m[50:60]) == bytes(range(50, 60))


def test_io_words_are_written_even_for_empty_slices():
    # base/tests/integration.rs:2915-3015
    b = py_base.Base(py_base.Setup("", 64, IO, b"\xff" * 64))
    b.execute_into(py_base.Algorithm(0), b"", bytearray(0))
    m = bytes(b.memory())
    assert struct.unpack_from("<Q", m, 16)[0] == 0 and struct.unpack_from("<Q", m, 32)[0] == 0
    data, out = b"abcdef", bytearray(10)
    b.execute_into(py_base.Algorithm(0), data, out)
    m = bytes(b.memory())
    assert struct.unpack_from("<Q", m, 16)[0] == 6 and struct.unpack_from("<Q", m, 32)[0] == 10
    assert struct.unpack_from("<Q", m, 8)[0] != 0 and struct.unpack_from("<Q", m, 24)[0] != 0
    assert m[40:] == b"\xff" * 24


def test_clif_text_is_a_parse_error():
    # base/tests/integration.rs:2413-2457 expects Error::ClifParse for bad IR;
    # here all CLIF is unparsable by construction.
    with pytest.raises(ValueError, match="ClifParse"):
        py_base.Base(py_base.Setup("function u0:0(i64) system_v {\nblock0(v0: i64):\n return\n}", 64, IO))
    with pytest.raises(ValueError, match="unknown native plugin"):
        py_base.Base(py_base.Setup("native:nope", 64, py_base.IoOffsets(**py_base.DEFAULT_IO)))
    with pytest.raises(ValueError, match="io_offsets"):
        py_base.Base(py_base.Setup("native:moe_ffn", 64, IO))


def test_native_plugin_stage_table():
    art = py_base.native_artifact("moe_ffn")
    assert art.setup.cranelift_ir == "native:moe_ffn"
    assert art.main.fn_idx == 1                      # fn 0 is the no-op stub (FFI.lean:652-654)
    for name in ("prep", "infer", "stack", "fetchTopk", "fetchDequant"):
        assert name in art.extras
    b = py_base.Base(art.setup)
    b.execute(py_base.Algorithm(0))                  # stub
    with pytest.raises(RuntimeError, match="out of range"):
        b.execute(py_base.Algorithm(99))
    with pytest.raises(RuntimeError, match="payload shorter than header"):
        b.execute(art.main, b"abc")
    with pytest.raises(RuntimeError, match="load has not run"):
        b.execute(art.extras["prep"], b"\0" * 16)
    b.close()


def test_artifact_json_roundtrip_and_errors(tmp_path):
    art = py_base.native_artifact("moe_ffn")
    art.setup.initial_memory = bytes([1, 2, 3, 255])
    p = tmp_path / "a.json"
    p.write_text(art.to_json())
    back = py_base.load_artifact(p)
    assert back.setup.cranelift_ir == art.setup.cranelift_ir
    assert back.setup.initial_memory == bytes([1, 2, 3, 255])
    assert back.setup.io_offsets == art.setup.io_offsets
    assert {k: v.fn_idx for k, v in back.extras.items()} == {k: v.fn_idx for k, v in art.extras.items()}
    # serde defaults: initial_memory and extras may be omitted (base-types/src/lib.rs:38-39, 52-53)
    d = json.loads(art.to_json())
    del d["setup"]["initial_memory"], d["extras"]
    a3 = py_base.loads_artifact(json.dumps(d))
    assert a3.setup.initial_memory == b"" and a3.extras == {}
    # missing fields are errors (py-base/tests/test_base.py style)
    for path in (("setup",), ("main",), ("setup", "memory_size"), ("setup", "io_offsets"), ("main", "fn_idx")):
        d2 = json.loads(art.to_json())
        t = d2
        for k in path[:-1]:
            t = t[k]
        del t[path[-1]]
        with pytest.raises(ValueError):
            py_base.loads_artifact(json.dumps(d2))
    with pytest.raises(ValueError):
        py_base.loads_artifact("{not json")
    d4 = json.loads(art.to_json())
    d4["setup"]["initial_memory"] = [256]
    with pytest.raises(ValueError):
        py_base.loads_artifact(json.dumps(d4))


def _bincode_artifact(ir: bytes, mem_size, io, init: bytes, main_fn, extras):
    def s(b):
        return struct.pack("<Q", len(b)) + b

    def alg(fn):
        return struct.pack("<I", fn) + struct.pack("<Q", 0)
    out = s(ir) + struct.pack("<Q", mem_size) + struct.pack("<4Q", *io) + s(init) + alg(main_fn)
    out += struct.pack("<Q", len(extras))
    for k, fn in extras:
        out += s(k.encode()) + alg(fn)
    return out


def test_artifact_from_bincode_bytes():
    raw = _bincode_artifact(b"native:moe_ffn", 4096, (0x18, 0x20, 0x28, 0x30), b"\x01\x02", 1,
                            [("prep", 2), ("infer", 3)])
    a = py_base.artifact_from_bytes(raw)
    assert a.setup.cranelift_ir == "native:moe_ffn" and a.setup.memory_size == 4096
    assert a.setup.initial_memory == b"\x01\x02" and a.main.fn_idx == 1
    assert a.extras["infer"].fn_idx == 3
    with pytest.raises(ValueError):
        py_base.artifact_from_bytes(raw[:-3])


def test_run_helper():
    assert py_base.run(py_base.Setup("", 0, IO), py_base.Algorithm(0)) == []


def test_huge_memory_size_and_deep_json_are_errors_not_corruption():
    # memory_size near 2^64 must not wrap the allocation size; the reference aborts on such a resize
    # (base/src/lib.rs:36-52), here it is an Execution error
    for size in (2 ** 64 - 1, 2 ** 64 - 40, 2 ** 41):
        with pytest.raises((RuntimeError, ValueError, OverflowError)):
            py_base.Base(py_base.Setup("", size, IO))
    art = py_base.native_artifact("moe_ffn")
    d = json.loads(art.to_json())
    d["setup"]["memory_size"] = 2 ** 64 - 1            # representable as u64: parsed exactly, refused by Base
    a = py_base.loads_artifact(json.dumps(d))
    assert a.setup.memory_size == 2 ** 64 - 1
    with pytest.raises((RuntimeError, ValueError)):
        py_base.Base(a.setup)
    d["setup"]["memory_size"] = 2 ** 64                # not a u64
    with pytest.raises(ValueError):
        py_base.loads_artifact(json.dumps(d))
    with pytest.raises(ValueError):
        py_base.loads_artifact("[" * 100000 + "]" * 100000)
