"""Section A of the C ABI on a GPU: the calls a `hipml-cuda` crate makes where `hipml-hip`
calls amdhip64 (crates/hipml-hip/src/ffi.rs:29-105) -- memory, copies, events, streams,
stream capture + graph replay, and launching a kernel by its reference entry name with the
reference's own argument array (crates/hipml-kernels/src/launch/device/graph_launch.rs:
946-973)."""
import ctypes as C

import numpy as np
import pytest

import oracle as O
from tests import cases

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def lib():
    from hipml_b200 import _lib
    L = _lib.load()
    _lib.check("init", L.hipml_init(0))
    return L


def _ok(rc):
    from hipml_b200 import _lib
    _lib.check("call", rc)


def test_device_queries(lib):
    n = C.c_int()
    _ok(lib.hipml_get_device_count(C.byref(n)))
    assert n.value >= 1
    dev = C.c_int(-1)
    _ok(lib.hipml_get_device(C.byref(dev), 0))
    _ok(lib.hipml_set_device(dev.value))
    name = C.create_string_buffer(128)
    _ok(lib.hipml_device_get_name(name, 128, dev.value))
    assert name.value
    total, free = C.c_size_t(), C.c_size_t()
    _ok(lib.hipml_device_total_mem(C.byref(total), dev.value))
    _ok(lib.hipml_mem_get_info(C.byref(free), C.byref(total)))
    assert 0 < free.value <= total.value
    major, minor = C.c_int(), C.c_int()
    _ok(lib.hipml_device_compute_capability(C.byref(major), C.byref(minor), dev.value))
    assert major.value == 10
    assert lib.hipml_get_device(C.byref(dev), 10_000) != 0


def test_memory_copies_events_and_streams(lib):
    n = 1 << 20
    host = np.arange(n, dtype=np.float32)
    back = np.zeros_like(host)
    a, b = C.c_void_p(), C.c_void_p()
    _ok(lib.hipml_malloc(C.byref(a), host.nbytes))
    _ok(lib.hipml_malloc(C.byref(b), host.nbytes))
    _ok(lib.hipml_memset(b, 0, host.nbytes))
    stream, e0, e1 = C.c_void_p(), C.c_void_p(), C.c_void_p()
    _ok(lib.hipml_stream_create(C.byref(stream)))
    _ok(lib.hipml_event_create(C.byref(e0)))
    _ok(lib.hipml_event_create(C.byref(e1)))
    _ok(lib.hipml_memcpy(a, host.ctypes.data_as(C.c_void_p), host.nbytes, 1))
    _ok(lib.hipml_event_record(e0, stream))
    _ok(lib.hipml_memcpy_async(b, a, host.nbytes, 3, stream))
    _ok(lib.hipml_event_record(e1, stream))
    _ok(lib.hipml_stream_synchronize(stream))
    _ok(lib.hipml_event_synchronize(e1))
    ms = C.c_float(-1.0)
    _ok(lib.hipml_event_elapsed_time(C.byref(ms), e0, e1))
    assert ms.value >= 0.0
    _ok(lib.hipml_memcpy(back.ctypes.data_as(C.c_void_p), b, host.nbytes, 2))
    assert np.array_equal(back, host)
    # a second stream waits on an event of the first
    s2 = C.c_void_p()
    _ok(lib.hipml_stream_create(C.byref(s2)))
    _ok(lib.hipml_stream_wait_event(s2, e1, 0))
    _ok(lib.hipml_stream_synchronize(s2))
    pinned = C.c_void_p()
    _ok(lib.hipml_host_alloc(C.byref(pinned), 4096))
    _ok(lib.hipml_host_free(pinned))
    for h in (e0, e1):
        _ok(lib.hipml_event_destroy(h))
    for h in (stream, s2):
        _ok(lib.hipml_stream_destroy(h))
    _ok(lib.hipml_free(a))
    _ok(lib.hipml_free(b))
    _ok(lib.hipml_device_synchronize())


def test_launch_by_reference_entry_name_and_graph_replay(lib):
    """kv_encode_q8 through Module::kernel(name) + Kernel::launch's pointer array, captured in
    a graph; the position comes from the device step buffer, so one graph serves two steps."""
    c = cases.KV_ENCODE_CASE
    n_kv, hd, seq = c["n_kv"], c["head_dim"], c["seq"]
    k, v = cases.kv_encode_case_inputs()
    row = hd // 32 * 34
    nbytes = n_kv * seq * row
    dk, dv, kc, vc, step = (C.c_void_p() for _ in range(5))
    for ptr, size in ((dk, k.nbytes), (dv, v.nbytes), (kc, nbytes), (vc, nbytes), (step, 32)):
        _ok(lib.hipml_malloc(C.byref(ptr), size))
    _ok(lib.hipml_memcpy(dk, k.ctypes.data_as(C.c_void_p), k.nbytes, 1))
    _ok(lib.hipml_memcpy(dv, v.ctypes.data_as(C.c_void_p), v.nbytes, 1))
    _ok(lib.hipml_memset(kc, 0xAB, nbytes))
    _ok(lib.hipml_memset(vc, 0xAB, nbytes))

    module, fn = C.c_void_p(), C.c_void_p()
    _ok(lib.hipml_module_load(C.byref(module), b"hipml.co"))
    _ok(lib.hipml_module_get_function(C.byref(fn), module, b"kv_encode_q8"))
    v_hd, v_stride = C.c_int(hd), C.c_int(seq)
    args = [dk, dv, kc, vc, v_hd, v_stride, step]
    params = (C.c_void_p * len(args))(*[C.cast(C.pointer(a), C.c_void_p) for a in args])

    stream, graph, exe = C.c_void_p(), C.c_void_p(), C.c_void_p()
    _ok(lib.hipml_stream_create(C.byref(stream)))
    _ok(lib.hipml_stream_begin_capture(stream, 0))
    _ok(lib.hipml_module_launch_kernel(fn, n_kv, 1, 1, hd, 1, 1, 0, stream, params, None))
    _ok(lib.hipml_stream_end_capture(stream, C.byref(graph)))
    _ok(lib.hipml_graph_instantiate(C.byref(exe), graph, None, None, 0))
    _ok(lib.hipml_graph_upload(exe, stream))
    krows, vrows = cases.kv_encode_expected_bytes(k, v, n_kv, hd)
    want = np.full((n_kv, seq, row), 0xAB, dtype=np.uint8)
    for pos in (3, 6):
        st = np.array([pos, pos + 1, 0, 0, 0, 0, 0, 0], dtype=np.int32)
        _ok(lib.hipml_memcpy_async(step, st.ctypes.data_as(C.c_void_p), 32, 1, stream))
        _ok(lib.hipml_graph_launch(exe, stream))
        _ok(lib.hipml_stream_synchronize(stream))
        for h in range(n_kv):
            want[h, pos] = krows[h]
    got = np.zeros(nbytes, dtype=np.uint8)
    _ok(lib.hipml_memcpy(got.ctypes.data_as(C.c_void_p), kc, nbytes, 2))
    assert np.array_equal(got.reshape(n_kv, seq, row), want)
    assert O.compare(O.dequantize_q8(want[:, 3].ravel()), O.dequantize_q8(np.concatenate(krows))) == (0.0, 0.0)
    _ok(lib.hipml_graph_exec_destroy(exe))
    _ok(lib.hipml_graph_destroy(graph))
    _ok(lib.hipml_stream_destroy(stream))
    _ok(lib.hipml_module_unload(module))
    for ptr in (dk, dv, kc, vc, step):
        _ok(lib.hipml_free(ptr))
