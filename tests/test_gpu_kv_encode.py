"""KV append/quantise kernels against the host format definition: bit-exact bytes.

Mirrors the reference's `kv_encode_q8` device-parity case (crates/hipml-core/src/parity.rs:
364-378, tolerance EXACT) and widens it to the shipped shape, the bulk and per-slot forms,
edge values and a canary check that no byte outside the target rows is written.
"""
import numpy as np
import pytest
import torch

import oracle as O
from tests import cases

pytestmark = pytest.mark.gpu

CANARY = 0xAB


def _dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a))
    if dtype is not None:
        t = t.to(dtype)
    return t.cuda()


def _cache(n_bytes):
    return torch.full((n_bytes,), CANARY, dtype=torch.uint8, device="cuda")


def _step(pos, seq=None):
    seq = pos + 1 if seq is None else seq
    return torch.tensor([pos, seq, 0, 0, 0, 0, 0, 0], dtype=torch.int32, device="cuda")


def _expect_rows(cache_np, rows_by_head, n_kv, stride, pos, row_bytes, base=0):
    """Every byte of `cache_np` is the canary except the rows at `pos`, which match."""
    want = np.full_like(cache_np, CANARY)
    for h in range(n_kv):
        at = base + (h * stride + pos) * row_bytes
        want[at:at + row_bytes] = rows_by_head[h]
    return want


def test_reference_case_kv_encode_q8_is_bit_exact():
    from hipml_b200 import api
    c = cases.KV_ENCODE_CASE
    n_kv, hd, seq, pos = c["n_kv"], c["head_dim"], c["seq"], c["pos"]
    k, v = cases.kv_encode_case_inputs()
    row_bytes = hd // 32 * 34
    kc, vc = _cache(n_kv * seq * row_bytes), _cache(n_kv * seq * row_bytes)
    api.kv_encode(_step(pos), _dev(k), _dev(v), kc, vc, n_kv, hd, seq)
    torch.cuda.synchronize()
    krows, vrows = cases.kv_encode_expected_bytes(k, v, n_kv, hd)
    assert np.array_equal(kc.cpu().numpy(), _expect_rows(kc.cpu().numpy(), krows, n_kv, seq, pos, row_bytes))
    assert np.array_equal(vc.cpu().numpy(), _expect_rows(vc.cpu().numpy(), vrows, n_kv, seq, pos, row_bytes))
    # the reference compares decoded values at Tol::EXACT: same thing, stated its way
    got = O.dequantize_q8(kc.cpu().numpy().reshape(n_kv, seq, row_bytes)[:, pos].ravel())
    want = O.dequantize_q8(np.concatenate(krows))
    assert O.compare(want, got) == (0.0, 0.0)


@pytest.mark.parametrize("hd", [32, 64, 96, 256])
def test_single_row_shapes_and_edge_values(hd):
    from hipml_b200 import api
    n_kv, stride, pos = 4, 11, 7
    rng = O.Rng(0x51 + hd)
    k = rng.normals(n_kv * hd, 2.0)
    v = rng.normals(n_kv * hd, 0.01)
    # a zero block, an exact half-way code (x*id = 0.5 -> rounds away from zero), a huge
    # value, a tiny block whose scale is an f16 subnormal, and a NaN (encodes as code 0)
    k[0:32] = 0.0
    if hd >= 64:
        k[32:64] = 0.0
        k[32] = 127.0
        k[33] = 0.5
        k[34] = -0.5
        k[35] = 1.5
    v[0:32] = 1e-7
    v[5] = 3e-7
    if hd >= 64:
        v[32:64] = np.float32(1e30)
        v[40] = np.float32(np.nan)
    if hd >= 96:
        k[64:96] = np.float32(np.nan)   # a block of NaNs only: scale 0, codes 0
    row_bytes = hd // 32 * 34
    kc, vc = _cache(n_kv * stride * row_bytes), _cache(n_kv * stride * row_bytes)
    api.kv_encode(_step(pos), _dev(k), _dev(v), kc, vc, n_kv, hd, stride)
    torch.cuda.synchronize()
    krows, vrows = cases.kv_encode_expected_bytes(k, v, n_kv, hd)
    assert np.array_equal(kc.cpu().numpy(), _expect_rows(kc.cpu().numpy(), krows, n_kv, stride, pos, row_bytes))
    assert np.array_equal(vc.cpu().numpy(), _expect_rows(vc.cpu().numpy(), vrows, n_kv, stride, pos, row_bytes))


@pytest.mark.parametrize("misaligned", [False, True], ids=["warp_per_row", "reference_shape"])
def test_bulk_rows_land_at_start_plus_r_from_src0_plus_r(misaligned):
    from hipml_b200 import api
    n_kv, hd, stride = 4, 256, 300
    start, src0, rows, total = 37, 5, 130, 140
    rng = O.Rng(0xB01C)
    k = rng.normals(total * n_kv * hd).reshape(total, n_kv, hd)
    v = rng.normals(total * n_kv * hd, 3.0).reshape(total, n_kv, hd)
    # edge values inside the copied rows: zero block, half-way codes, huge, subnormal scale,
    # one NaN, a block of NaNs only
    k[src0 + 1, 0, 0:32] = 0.0
    k[src0 + 1, 1, 32:64] = 0.0
    k[src0 + 1, 1, 32:36] = (127.0, 0.5, -0.5, 1.5)
    v[src0 + 2, 2, 64:96] = np.float32(1e30)
    v[src0 + 2, 2, 70] = np.float32(np.nan)
    v[src0 + 3, 3, 0:32] = np.float32(1e-7)
    k[src0 + 4, 3, 224:256] = np.float32(np.nan)
    row_bytes = 272
    kc, vc = _cache(n_kv * stride * row_bytes), _cache(n_kv * stride * row_bytes)
    kd, vd = _dev(k), _dev(v)
    if misaligned:
        # sources 4 bytes off a 16-byte boundary take the kernel with the reference's launch shape
        kd = torch.cat([kd.new_zeros(1), kd.flatten()])[1:]
        vd = torch.cat([vd.new_zeros(1), vd.flatten()])[1:]
        assert kd.data_ptr() % 16 == 4
    api.kv_encode_bulk(kd, vd, kc, vc, n_kv, hd, stride, start, src0, rows)
    torch.cuda.synchronize()
    for src, cache in ((k, kc), (v, vc)):
        want = np.full((n_kv, stride, row_bytes), CANARY, dtype=np.uint8)
        for h in range(n_kv):
            want[h, start:start + rows] = O.quantize_q8(src[src0:src0 + rows, h]).reshape(rows, row_bytes)
        assert np.array_equal(cache.cpu().numpy().reshape(n_kv, stride, row_bytes), want)


def test_bulk_full_chunk_2048_rows_matches_host_encode():
    from hipml_b200 import api
    n_kv, hd, stride, rows, start = 4, 256, 8200, 2048, 4096
    g = torch.Generator(device="cuda").manual_seed(1)
    k = torch.randn(rows, n_kv * hd, device="cuda", generator=g)
    v = torch.randn(rows, n_kv * hd, device="cuda", generator=g)
    kc = torch.zeros(n_kv * stride * 272, dtype=torch.uint8, device="cuda")
    vc = torch.zeros_like(kc)
    api.kv_encode_bulk(k, v, kc, vc, n_kv, hd, stride, start, 0, rows)
    torch.cuda.synchronize()
    for src, cache in ((k, kc), (v, vc)):
        host = src.cpu().numpy().reshape(rows, n_kv, hd)
        got = cache.cpu().numpy().reshape(n_kv, stride, 272)
        for h in range(n_kv):
            want = O.quantize_q8(host[:, h]).reshape(rows, 272)
            assert np.array_equal(got[h, start:start + rows], want)
        assert not got[:, :start].any() and not got[:, start + rows:].any()


@pytest.mark.parametrize("slots", [1, 8, 16])
def test_per_slot_rows_use_the_slot_offset_and_its_own_position(slots):
    from hipml_b200 import api
    n_kv, hd, stride = 4, 256, 64
    row_bytes, slot_bytes = 272, 4 * 64 * 272
    rng = O.Rng(0x5107 + slots)
    k = rng.normals(slots * n_kv * hd).reshape(slots, n_kv, hd)
    v = rng.normals(slots * n_kv * hd).reshape(slots, n_kv, hd)
    positions = [(7 * s + 3) % stride for s in range(slots)]
    pos = torch.tensor([[p, p + 1] for p in positions], dtype=torch.int32, device="cuda")
    kc, vc = _cache(slots * slot_bytes), _cache(slots * slot_bytes)
    api.kv_encode_rows(_dev(k), _dev(v), kc, vc, n_kv, hd, stride, pos, slot_bytes, slots)
    torch.cuda.synchronize()
    for src, cache in ((k, kc), (v, vc)):
        want = np.full((slots, n_kv, stride, row_bytes), CANARY, dtype=np.uint8)
        for s in range(slots):
            for h in range(n_kv):
                want[s, h, positions[s]] = O.quantize_q8(src[s, h])
        assert np.array_equal(cache.cpu().numpy().reshape(slots, n_kv, stride, row_bytes), want)


def test_f32_append_single_row_and_chunk():
    from hipml_b200 import api
    n_ctx, width = 50, 1024
    rng = O.Rng(0xF32A)
    base_k = rng.normals(n_ctx * width).reshape(n_ctx, width)
    base_v = rng.normals(n_ctx * width).reshape(n_ctx, width)
    k_row, v_row = rng.normals(width), rng.normals(width)
    kc, vc = _dev(base_k), _dev(base_v)
    api.kv_append_f32(_step(17), kc, vc, _dev(k_row), _dev(v_row), width)
    want_k, want_v = base_k.copy(), base_v.copy()
    want_k[17], want_v[17] = k_row, v_row
    assert np.array_equal(kc.cpu().numpy(), want_k) and np.array_equal(vc.cpu().numpy(), want_v)
    tok, pos0 = 9, 30
    k, v = rng.normals(tok * width).reshape(tok, width), rng.normals(tok * width).reshape(tok, width)
    api.kv_append_chunk_f32(kc, vc, _dev(k), _dev(v), pos0, width, tok)
    want_k[pos0:pos0 + tok], want_v[pos0:pos0 + tok] = k, v
    assert np.array_equal(kc.cpu().numpy(), want_k) and np.array_equal(vc.cpu().numpy(), want_v)
    # odd width takes the scalar copy path
    w2 = 33
    kc2 = torch.zeros(10, w2, device="cuda")
    vc2 = torch.zeros(10, w2, device="cuda")
    k2, v2 = rng.normals(3 * w2).reshape(3, w2), rng.normals(3 * w2).reshape(3, w2)
    api.kv_append_chunk_f32(kc2, vc2, _dev(k2), _dev(v2), 4, w2, 3)
    assert np.array_equal(kc2.cpu().numpy()[4:7], k2) and np.array_equal(vc2.cpu().numpy()[4:7], v2)
    assert not kc2.cpu().numpy()[:4].any() and not kc2.cpu().numpy()[7:].any()


def test_argument_errors_use_the_reference_messages():
    from hipml_b200 import api, _lib
    z = torch.zeros(1024, device="cuda")
    c = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    with pytest.raises(_lib.HipmlError, match="unknown KV dtype 7"):
        api.kv_encode(_step(0), z, z, c, c, 4, 64, 8, dtype=7)
    with pytest.raises(_lib.HipmlError, match="unknown KV dtype -1"):
        api.kv_encode(_step(0), z, z, c, c, 4, 64, 8, dtype=-1)
    with pytest.raises(_lib.HipmlError, match="head_dim 48"):
        api.kv_encode(_step(0), z, z, c, c, 4, 48, 8)
