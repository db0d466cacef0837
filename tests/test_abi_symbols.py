"""The C-ABI library loads without a GPU and exports every symbol the header declares."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "hipml_cuda.h")


def _declared():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(hipml_[a-z0-9_]+)\s*\(", text)))


def _lib():
    import __graft_entry__ as entry
    entry.build()
    from hipml_b200 import _lib as L
    return L


def test_header_declares_the_expected_groups():
    names = _declared()
    for must in ["hipml_init", "hipml_malloc", "hipml_memcpy_async", "hipml_stream_begin_capture",
                 "hipml_module_launch_kernel", "hipml_kv_encode", "hipml_kv_encode_bulk",
                 "hipml_kv_encode_rows", "hipml_kv_append_f32", "hipml_attn_decode_kv",
                 "hipml_attn_decode_rows", "hipml_attn_decode_batch", "hipml_attn_chunk"]:
        assert must in names


def test_library_exports_every_declared_symbol():
    L = _lib()
    lib = L.load()
    missing = [n for n in _declared() if not hasattr(lib, n)]
    assert not missing, f"declared but not exported: {missing}"


def test_python_prototypes_cover_the_header():
    L = _lib()
    assert sorted(L.SIGNATURES) == _declared()


def test_rust_binding_is_in_step_with_the_header():
    """hipml_b200/host/hipml-cuda/src/ffi.rs is generated from the header (no Rust toolchain
    exists where this library is built): the committed file must be what the generator writes,
    with one declaration per symbol."""
    import importlib.util
    crate = os.path.join(ROOT, "hipml_b200", "host", "hipml-cuda")
    spec = importlib.util.spec_from_file_location("gen_ffi", os.path.join(crate, "gen_ffi.py"))
    gen = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(gen)
    text = open(os.path.join(crate, "src", "ffi.rs")).read()
    assert text == gen.render()
    assert sorted(re.findall(r"pub fn (hipml_[a-z0-9_]+)\(", text)) == _declared()


def test_calls_that_need_no_gpu():
    L = _lib()
    lib = L.load()
    assert lib.hipml_version().decode().startswith("hipml_cuda")
    assert b"invalid argument" in lib.hipml_get_error_string(L.ERR_INVALID_ARGUMENT)
    # 24/4/256 at 100,000 keys: four f16 planes of n_kv * roundup(keys, 128) * 256
    assert lib.hipml_attn_chunk_workspace_bytes(4, 256, 97952, 2048) == 4 * 4 * 100096 * 256 * 2
    assert lib.hipml_attn_chunk_workspace_bytes(4, 64, 0, 16) == 0
    mod = C.c_void_p()
    assert lib.hipml_module_load(C.byref(mod), None) == 0
    fn = C.c_void_p()
    for name in [b"kv_encode_q8", b"kv_encode_bulk_q8", b"kv_encode_q8_b", b"kv_append_f32",
                 b"kv_append_chunk_f32", b"attn_decode_kv_reduce", b"attn_decode_kv_reduce_b",
                 b"attn_chunk_combine_f32"]:
        assert lib.hipml_module_get_function(C.byref(fn), mod, name) == 0 and fn.value
    rc = lib.hipml_module_get_function(C.byref(fn), mod, b"no_such_kernel")
    assert rc == L.ERR_UNKNOWN_KERNEL
    assert b"no_such_kernel" in lib.hipml_last_error_message()
    with pytest.raises(L.HipmlError, match=r"lookup failed: 10002 \(kernel no_such_kernel"):
        L.check("lookup", rc)


def test_split_policies_match_the_reference_tables():
    from hipml_b200 import api
    # deep_kv.rs:102-110 -> 84 / 128 / 256 / 256 at the bench depths
    assert [api.decode_splits(s) for s in (672, 8192, 32768, 100000)] == [84, 128, 256, 256]
    assert api.decode_splits(1) == 1 and api.decode_splits(63) == 7
    # batch/kv.rs:39-42 -> 64 (B=8) / 32 (B=16) at stride 8192
    assert api.batch_splits(8192, 8) == 64 and api.batch_splits(8192, 16) == 32
    assert api.batch_splits(32768, 1) == 256 and api.batch_splits(10, 4) == 1
    # attn_tile.rs:138-151
    assert api.prefill_splits(0) == 1 and api.prefill_splits(8191) == 1
    assert api.prefill_splits(8192) == 8
