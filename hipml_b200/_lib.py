"""ctypes binding of libhipml_cuda.so, the C-ABI library declared in include/hipml_cuda.h.

The library is built in-tree (``python hipml_b200/build.py``). There is no fallback:
if it cannot be loaded, importing the product path raises.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "lib", "libhipml_cuda.so")

ERR_BASE = 10000
ERR_INVALID_ARGUMENT = 10001
ERR_UNKNOWN_KERNEL = 10002
ERR_WORKSPACE = 10003
ERR_DEVICE_STATUS = 10004

_vp, _i, _f, _sz, _u = C.c_void_p, C.c_int, C.c_float, C.c_size_t, C.c_uint

# name -> (restype, argtypes); must list every symbol include/hipml_cuda.h declares.
SIGNATURES = {
    # A. device layer
    "hipml_init": (_i, [_u]),
    "hipml_get_device_count": (_i, [C.POINTER(_i)]),
    "hipml_get_device": (_i, [C.POINTER(_i), _i]),
    "hipml_set_device": (_i, [_i]),
    "hipml_device_get_name": (_i, [C.c_char_p, _i, _i]),
    "hipml_device_total_mem": (_i, [C.POINTER(_sz), _i]),
    "hipml_device_compute_capability": (_i, [C.POINTER(_i), C.POINTER(_i), _i]),
    "hipml_get_error_string": (C.c_char_p, [_i]),
    "hipml_last_error_message": (C.c_char_p, []),
    "hipml_malloc": (_i, [C.POINTER(_vp), _sz]),
    "hipml_free": (_i, [_vp]),
    "hipml_memset": (_i, [_vp, _i, _sz]),
    "hipml_mem_get_info": (_i, [C.POINTER(_sz), C.POINTER(_sz)]),
    "hipml_memcpy": (_i, [_vp, _vp, _sz, _i]),
    "hipml_memcpy_async": (_i, [_vp, _vp, _sz, _i, _vp]),
    "hipml_device_synchronize": (_i, []),
    "hipml_host_alloc": (_i, [C.POINTER(_vp), _sz]),
    "hipml_host_free": (_i, [_vp]),
    "hipml_event_create": (_i, [C.POINTER(_vp)]),
    "hipml_event_destroy": (_i, [_vp]),
    "hipml_event_record": (_i, [_vp, _vp]),
    "hipml_event_synchronize": (_i, [_vp]),
    "hipml_event_elapsed_time": (_i, [C.POINTER(_f), _vp, _vp]),
    "hipml_stream_create": (_i, [C.POINTER(_vp)]),
    "hipml_stream_destroy": (_i, [_vp]),
    "hipml_stream_synchronize": (_i, [_vp]),
    "hipml_stream_wait_event": (_i, [_vp, _vp, _u]),
    "hipml_stream_begin_capture": (_i, [_vp, _i]),
    "hipml_stream_end_capture": (_i, [_vp, C.POINTER(_vp)]),
    "hipml_graph_instantiate": (_i, [C.POINTER(_vp), _vp, _vp, C.c_char_p, _sz]),
    "hipml_graph_launch": (_i, [_vp, _vp]),
    "hipml_graph_upload": (_i, [_vp, _vp]),
    "hipml_graph_destroy": (_i, [_vp]),
    "hipml_graph_exec_destroy": (_i, [_vp]),
    "hipml_module_load": (_i, [C.POINTER(_vp), C.c_char_p]),
    "hipml_module_unload": (_i, [_vp]),
    "hipml_module_get_function": (_i, [C.POINTER(_vp), _vp, C.c_char_p]),
    "hipml_module_launch_kernel": (_i, [_vp, _u, _u, _u, _u, _u, _u, _u, _vp, C.POINTER(_vp), _vp]),
    # B. launchers
    "hipml_kv_encode": (_i, [_vp, _vp, _i, _vp, _vp, _vp, _vp, _i, _i, _i]),
    "hipml_kv_encode_bulk": (_i, [_vp, _i, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i]),
    "hipml_kv_encode_rows": (_i, [_vp, _i, _vp, _vp, _vp, _vp, _i, _i, _i, _vp, _i, _i]),
    "hipml_kv_append_f32": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i]),
    "hipml_kv_append_chunk_f32": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i]),
    "hipml_attn_decode_kv": (_i, [_vp, _vp, _i, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _f,
                                  _i, _sz, _sz]),
    "hipml_attn_decode_cols": (_i, [_vp, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _f, _i,
                                    _i, _i, _i, _i]),
    "hipml_kv_rows_copy": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _i]),
    "hipml_attn_decode_kv_gated": (_i, [_vp, _vp, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i,
                                        _f, _i, _sz, _sz]),
    "hipml_attn_decode_kv_append": (_i, [_vp, _vp, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i,
                                         _i, _i, _f, _i, _sz, _sz]),
    "hipml_attn_decode_batch_append": (_i, [_vp, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i,
                                            _i, _i, _f, _i, _i, _i, _i, _i, _i]),
    "hipml_attn_decode_kv_shard": (_i, [_vp, _vp, _i, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i,
                                        _f, _i, _sz, _sz]),
    "hipml_attn_decode_combine": (_i, [_vp, _vp, _vp, _i, _i, _i]),
    "hipml_attn_front": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, C.POINTER(_i), _vp,
                              _f, _f]),
    "hipml_qg_split_chunk": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i]),
    "hipml_norm_rope_chunk": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _f, _f, _i, _i]),
    "hipml_q_gate": (_i, [_vp, _vp, _vp, _vp, C.c_longlong]),
    "hipml_attn_front_append_q8": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i,
                                        _i, _i, C.POINTER(_i), _vp, _vp, _i, _i, _i, _f, _f]),
    "hipml_decode_exchange_bytes": (_sz, [_i, _i, _i]),
    "hipml_attn_decode_kv_shard_exchange": (_i, [_vp, _vp, _i, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i,
                                                 _i, _i, _f, _i, _sz, _sz, C.POINTER(_vp), _i, _i,
                                                 _i, _u]),
    "hipml_attn_decode_kv_shard_exchange_append": (_i, [_vp, _vp, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp,
                                                        _vp, _i, _i, _i, _i, _f, _i, _sz, _sz,
                                                        C.POINTER(_vp), _i, _i, _i, _u]),
    "hipml_set_decode_cta_slots": (_i, [_i]),
    "hipml_set_decode_fold_mode": (_i, [_i]),
    "hipml_set_decode_body": (_i, [_i]),
    "hipml_decode_plan_quota": (_i, [C.POINTER(_i), _i, _i, _i, _i]),
    "hipml_attn_decode_kv_static": (_i, [_vp, _vp, _i, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _f, _i,
                                         _sz, _sz]),
    "hipml_attn_decode_cols_f32": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i]),
    "hipml_kv_append_cols_f32": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i]),
    "hipml_attn_decode_rows": (_i, [_vp, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _f,
                                    _i, _i, _i, _i, _i, _i]),
    "hipml_attn_decode_batch": (_i, [_vp, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i,
                                     _f, _i, _i, _i, _i, _i, _i, _i]),
    "hipml_attn_chunk_workspace_bytes": (_sz, [_i, _i, _i, _i]),
    "hipml_attn_chunk": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp, _vp, _i,
                              _i, _vp, _sz]),
    "hipml_attn_chunk_stage": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp, _sz]),
    "hipml_attn_chunk_staged": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _i, _vp, _vp, _i, _i, _i, _vp,
                                     _sz]),
    "hipml_attn_chunk_staged_gated": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp, _vp, _i, _i,
                                           _i, _vp, _sz]),
    "hipml_check_device_status": (_i, [_vp, C.POINTER(_i)]),
    "hipml_version": (C.c_char_p, []),
}

_lib = None


class HipmlError(RuntimeError):
    """A non-zero status from the C ABI; ``code`` is the int the call returned."""

    def __init__(self, what: str, code: int, text: str):
        super().__init__(f"{what} failed: {code} ({text})")
        self.code = code
        self.text = text


def load() -> C.CDLL:
    """Load the library and set every prototype. Raises if it is missing."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python hipml_b200/build.py` "
                "(there is no CPU or PyTorch fallback for the attention path)")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def check(what: str, code: int) -> None:
    """Mirror of hipml-hip's error wrapper: "{what} failed: {code} ({text})"."""
    if code == 0:
        return
    lib = load()
    if code >= ERR_BASE:
        text = lib.hipml_last_error_message().decode()
    else:
        text = lib.hipml_get_error_string(code).decode()
    raise HipmlError(what, code, text)
