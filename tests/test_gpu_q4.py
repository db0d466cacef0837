"""The q4_0 KV cache through every entry that takes a cache dtype: append/quantise (bit-exact
bytes), single-stream decode, multi-slot decode and chunk attention.

Reference: crates/hipml-core/src/kv.rs:36-90 (format: 18-byte blocks, scale = -vmax/8 of the
first element of largest magnitude, byte j = value j | value j+16 << 4), crates/hipml-core/src/
parity_kv.rs:118-215,232-246 (the q4 decode cases and the 100,000-row case), crates/
hipml-kernels/src/launch/device/batch_launch.rs:75,245 (per-slot encode and decode by dtype),
crates/hipml-kernels/src/attn_gpu/imp/attn_chunk_kv.rs:129-305 (chunk attention, dtype 2).
"""
import numpy as np
import pytest
import torch

import oracle as O
from tests import cases

pytestmark = pytest.mark.gpu

CANARY = 0xAB
Q4 = 1


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _step(pos, seq=None):
    seq = pos + 1 if seq is None else seq
    return torch.tensor([pos, seq, 0, 0, 0, 0, 0, 0], dtype=torch.int32, device="cuda")


def _cache(n_bytes):
    return torch.full((n_bytes,), CANARY, dtype=torch.uint8, device="cuda")


def _edge_rows(k, v, hd):
    """Edge values in the first blocks of a [.., hd] pair of rows (in place)."""
    k[..., 0:32] = 0.0                                   # zero block: scale -0.0, nibbles 8
    if hd >= 64:
        k[..., 32:64] = 0.0
        k[..., 34], k[..., 41] = 3.0, -3.0               # tie on |v|: the first one decides
        k[..., 35] = 0.1875                              # x*id = -0.5: rounds away from zero
        k[..., 36] = 2.9                                 # clamps at code 15
    v[..., 0:32] = 1e-7
    v[..., 5] = -3e-7                                    # scale is an f16 subnormal
    if hd >= 64:
        v[..., 32:64] = np.float32(1e30)                 # scale overflows f16
        v[..., 40] = np.float32(np.nan)                  # NaN never wins the max, encodes as 0
    if hd >= 96:
        k[..., 64:96] = np.float32(np.nan)               # a block of NaNs only


@pytest.mark.parametrize("hd", [32, 64, 96, 256])
def test_single_row_is_bit_exact_with_edge_values(hd):
    from hipml_b200 import api
    n_kv, stride, pos = 4, 11, 7
    rng = O.Rng(0x41 + hd)
    k = rng.normals(n_kv * hd, 2.0).reshape(n_kv, hd)
    v = rng.normals(n_kv * hd, 0.01).reshape(n_kv, hd)
    _edge_rows(k[1], v[2], hd)
    row = hd // 32 * 18
    kc, vc = _cache(n_kv * stride * row), _cache(n_kv * stride * row)
    api.kv_encode(_step(pos), _dev(k), _dev(v), kc, vc, n_kv, hd, stride, dtype=Q4)
    torch.cuda.synchronize()
    for src, cache in ((k, kc), (v, vc)):
        want = np.full((n_kv, stride, row), CANARY, dtype=np.uint8)
        for h in range(n_kv):
            want[h, pos] = O.quantize_q4(src[h])
        assert np.array_equal(cache.cpu().numpy().reshape(n_kv, stride, row), want)


@pytest.mark.parametrize("misaligned", [False, True], ids=["warp_per_row", "reference_shape"])
def test_bulk_rows_are_bit_exact(misaligned):
    from hipml_b200 import api
    n_kv, hd, stride, row = 4, 256, 300, 144
    start, src0, rows, total = 37, 5, 130, 140
    rng = O.Rng(0xB04C)
    k = rng.normals(total * n_kv * hd).reshape(total, n_kv, hd)
    v = rng.normals(total * n_kv * hd, 3.0).reshape(total, n_kv, hd)
    _edge_rows(k[src0 + 1, 1], v[src0 + 2, 2], hd)
    _edge_rows(k[src0 + rows - 1, 3], v[src0, 0], hd)
    kc, vc = _cache(n_kv * stride * row), _cache(n_kv * stride * row)
    kd, vd = _dev(k), _dev(v)
    if misaligned:
        kd = torch.cat([kd.new_zeros(1), kd.flatten()])[1:]
        vd = torch.cat([vd.new_zeros(1), vd.flatten()])[1:]
        assert kd.data_ptr() % 16 == 4
    api.kv_encode_bulk(kd, vd, kc, vc, n_kv, hd, stride, start, src0, rows, dtype=Q4)
    torch.cuda.synchronize()
    for src, cache in ((k, kc), (v, vc)):
        want = np.full((n_kv, stride, row), CANARY, dtype=np.uint8)
        for h in range(n_kv):
            want[h, start:start + rows] = O.quantize_q4(src[src0:src0 + rows, h]).reshape(rows, row)
        assert np.array_equal(cache.cpu().numpy().reshape(n_kv, stride, row), want)


def test_bulk_other_head_dim_takes_the_reference_shape():
    from hipml_b200 import api
    n_kv, hd, stride, row = 2, 64, 50, 36
    rng = O.Rng(0xB064)
    k = rng.normals(20 * n_kv * hd).reshape(20, n_kv, hd)
    v = rng.normals(20 * n_kv * hd).reshape(20, n_kv, hd)
    kc, vc = _cache(n_kv * stride * row), _cache(n_kv * stride * row)
    api.kv_encode_bulk(_dev(k), _dev(v), kc, vc, n_kv, hd, stride, 3, 0, 20, dtype=Q4)
    for src, cache in ((k, kc), (v, vc)):
        want = np.full((n_kv, stride, row), CANARY, dtype=np.uint8)
        for h in range(n_kv):
            want[h, 3:23] = O.quantize_q4(src[:, h]).reshape(20, row)
        assert np.array_equal(cache.cpu().numpy().reshape(n_kv, stride, row), want)


@pytest.mark.parametrize("slots", [1, 8])
def test_per_slot_rows_are_bit_exact(slots):
    from hipml_b200 import api
    n_kv, hd, stride, row = 4, 256, 64, 144
    slot_bytes = n_kv * stride * row
    rng = O.Rng(0x5147 + slots)
    k = rng.normals(slots * n_kv * hd).reshape(slots, n_kv, hd)
    v = rng.normals(slots * n_kv * hd).reshape(slots, n_kv, hd)
    positions = [(7 * s + 3) % stride for s in range(slots)]
    pos = torch.tensor([[p, p + 1] for p in positions], dtype=torch.int32, device="cuda")
    kc, vc = _cache(slots * slot_bytes), _cache(slots * slot_bytes)
    api.kv_encode_rows(_dev(k), _dev(v), kc, vc, n_kv, hd, stride, pos, slot_bytes, slots, dtype=Q4)
    for src, cache in ((k, kc), (v, vc)):
        want = np.full((slots, n_kv, stride, row), CANARY, dtype=np.uint8)
        for s in range(slots):
            for h in range(n_kv):
                want[s, h, positions[s]] = O.quantize_q4(src[s, h])
        assert np.array_equal(cache.cpu().numpy().reshape(slots, n_kv, stride, row), want)


def _run_decode(q, kb, vb, heads, n_kv, hd, seq, stride, scale, splits):
    from hipml_b200 import api
    out = torch.full((heads * hd,), float("nan"), device="cuda")
    acc = torch.full((heads * splits * hd,), float("nan"), device="cuda")
    ml = torch.full((heads * splits * 2,), float("nan"), device="cuda")
    api.attn_decode_kv(_step(seq - 1, seq), _dev(q), _dev(kb), _dev(vb), acc, ml, out, heads, n_kv,
                       hd, stride, scale, splits, selector=Q4)
    torch.cuda.synchronize()
    assert api.check_device_status() == 0
    return out.cpu().numpy(), acc.cpu().numpy(), ml.cpu().numpy()


def _assert_close(expected, got, tight=2e-5):
    assert np.all(np.isfinite(got))
    assert O.within(O.compare(expected, got), O.TOL_DEFAULT), O.compare(expected, got)
    ok, ma, rl = cases.attention_within_bar(expected, got)
    assert ok, (ma, rl)
    assert ma <= tight and rl <= tight, (ma, rl)


@pytest.mark.parametrize("case", cases.KV_CASES_Q4, ids=lambda c: c.name)
def test_reference_q4_cases(case):
    q, kb, vb = cases.kv_case_inputs(case)
    expected = cases.kv_case_expected(case, q, kb, vb)
    got, acc, ml = _run_decode(q, kb, vb, case.heads, case.n_kv, case.dim, case.seq, case.seq,
                               case.scale, case.splits)
    _assert_close(expected, got)
    assert not np.isnan(acc).any() and not np.isnan(ml).any()


def test_reference_deep_q4_case_100000_tokens():
    c = cases.DEEP_CASE_Q4
    q, kb, vb = cases.kv_case_inputs(c)
    expected = cases.kv_case_expected(c, q, kb, vb)
    got, _, _ = _run_decode(q, kb, vb, c.heads, c.n_kv, c.dim, c.seq, c.seq, c.scale, c.splits)
    _assert_close(expected, got)


def _poison_cache(n_kv, stride, hd):
    """Every block has a NaN scale: any row read by mistake poisons the output."""
    c = np.zeros((n_kv, stride, hd // 32, 18), dtype=np.uint8)
    c[..., 0], c[..., 1] = 0x00, 0x7E
    c[..., 2:] = 0x55
    return c.reshape(n_kv, stride, hd // 32 * 18)


@pytest.mark.parametrize("seq,pad", [(1, 7), (63, 1), (64, 0), (65, 200), (129, 0), (672, 136),
                                     (2500, 600)])
def test_shipped_shape_with_stride_beyond_live_length(seq, pad):
    from hipml_b200 import api
    heads, n_kv, hd, scale, row = 24, 4, 256, 0.0625, 144
    stride = seq + pad
    rng = O.Rng(0xD4 + seq)
    q = rng.normals(heads * hd)
    kc, vc = _poison_cache(n_kv, stride, hd), _poison_cache(n_kv, stride, hd)
    kc[:, :seq] = O.quantize_q4(rng.normals(n_kv * seq * hd)).reshape(n_kv, seq, row)
    vc[:, :seq] = O.quantize_q4(rng.normals(n_kv * seq * hd)).reshape(n_kv, seq, row)
    expected = O.attn_decode_kv(q, kc, vc, Q4, heads, n_kv, hd, seq, scale, stride=stride)
    got, _, _ = _run_decode(q, kc, vc, heads, n_kv, hd, seq, stride, scale, api.decode_splits(seq))
    _assert_close(expected, got)


def test_decode_reads_the_rows_the_encoder_wrote():
    """Append 70 rows with the bulk encoder and one with the single-row encoder, then decode:
    the device encode and the device decode agree on the format end to end."""
    from hipml_b200 import api
    heads, n_kv, hd, scale, stride, row = 24, 4, 256, 0.0625, 96, 144
    rng = O.Rng(0xE2E4)
    seq = 71
    k = rng.normals(seq * n_kv * hd).reshape(seq, n_kv * hd)
    v = rng.normals(seq * n_kv * hd).reshape(seq, n_kv * hd)
    q = rng.normals(heads * hd)
    kc, vc = _cache(n_kv * stride * row), _cache(n_kv * stride * row)
    api.kv_encode_bulk(_dev(k), _dev(v), kc, vc, n_kv, hd, stride, 0, 0, seq - 1, dtype=Q4)
    api.kv_encode(_step(seq - 1), _dev(k[seq - 1]), _dev(v[seq - 1]), kc, vc, n_kv, hd, stride,
                  dtype=Q4)
    kb = np.full((n_kv, stride, row), CANARY, dtype=np.uint8)
    vb = np.full((n_kv, stride, row), CANARY, dtype=np.uint8)
    kb[:, :seq] = O.quantize_q4(cases.pack_head_major(k, n_kv, seq, hd)).reshape(n_kv, seq, row)
    vb[:, :seq] = O.quantize_q4(cases.pack_head_major(v, n_kv, seq, hd)).reshape(n_kv, seq, row)
    assert np.array_equal(kc.cpu().numpy().reshape(n_kv, stride, row), kb)
    assert np.array_equal(vc.cpu().numpy().reshape(n_kv, stride, row), vb)
    expected = O.attn_decode_kv(q, kb, vb, Q4, heads, n_kv, hd, seq, scale, stride=stride)
    splits = api.decode_splits(seq)
    out = torch.full((heads * hd,), float("nan"), device="cuda")
    acc = torch.empty(heads * splits * hd, device="cuda")
    ml = torch.empty(heads * splits * 2, device="cuda")
    api.attn_decode_kv(_step(seq - 1, seq), _dev(q), kc, vc, acc, ml, out, heads, n_kv, hd, stride,
                       scale, splits, selector=Q4)
    _assert_close(expected, out.cpu().numpy())


@pytest.mark.parametrize("slots", [2, 8])
def test_multi_slot_decode_over_q4_caches(slots):
    from hipml_b200 import api
    heads, n_kv, hd, stride, row = 24, 4, 256, 2048, 144
    rng = O.Rng(0xBA74 + slots)
    depths = [100 + int(rng.uniform() * 1800) for _ in range(slots)]
    q = rng.normals(slots * heads * hd).reshape(slots, heads * hd)
    kc = np.stack([_poison_cache(n_kv, stride, hd) for _ in range(slots)])
    vc = np.stack([_poison_cache(n_kv, stride, hd) for _ in range(slots)])
    for s, d in enumerate(depths):
        kc[s, :, :d + 1] = O.quantize_q4(rng.normals(n_kv * (d + 1) * hd)).reshape(n_kv, d + 1, row)
        vc[s, :, :d + 1] = O.quantize_q4(rng.normals(n_kv * (d + 1) * hd)).reshape(n_kv, d + 1, row)
    splits = api.batch_splits(stride, slots)
    slot_bytes = n_kv * stride * row
    acc_slot, ml_slot, q_slot = heads * splits * hd, heads * splits * 2, heads * hd
    pos = torch.tensor([[d, d + 1] for d in depths], dtype=torch.int32, device="cuda")
    out = torch.full((slots, q_slot), float("nan"), device="cuda")
    acc = torch.full((slots * acc_slot,), float("nan"), device="cuda")
    ml = torch.full((slots * ml_slot,), float("nan"), device="cuda")
    api.attn_decode_batch(pos, _dev(q), _dev(kc), _dev(vc), acc, ml, out, heads, n_kv, hd, stride,
                          0.0625, splits, slot_bytes, acc_slot, ml_slot, q_slot, slots, 0, dtype=Q4)
    torch.cuda.synchronize()
    assert api.check_device_status() == 0
    got = out.cpu().numpy()
    for s, d in enumerate(depths):
        expected = O.attn_decode_kv(q[s], kc[s], vc[s], Q4, heads, n_kv, hd, d + 1, 0.0625,
                                    stride=stride)
        _assert_close(expected, got[s])


@pytest.mark.parametrize("mode,splits", [(0, 1), (0, 3), (2, 1), (2, 3), (3, 1)],
                         ids=["pair", "pair_split3", "scalar", "scalar_split3", "single_cta"])
def test_chunk_attention_over_a_q4_cache(mode, splits):
    """37 queries at position 29 (crates/hipml-cli/src/attn_chunk_parity.rs:124-207) over the
    same draws quantised as q4_0, with 11 unused rows behind the live ones."""
    from hipml_b200 import api
    c = cases.chunk_case_q8(pad=11, q4=True)
    want = cases.chunk_expected(c, threads=4)
    ws = torch.empty(api.attn_chunk_workspace_bytes(c.n_kv, c.hd, c.pos0, c.tok), dtype=torch.uint8,
                     device="cuda")
    out = torch.full((c.tok, c.heads * c.hd), float("nan"), device="cuda")
    qslots = (c.tok + 31) // 32 * 32
    pa = torch.empty(splits * qslots * c.heads * c.hd, device="cuda") if splits > 1 else None
    pm = torch.empty(splits * qslots * c.heads * 2, device="cuda") if splits > 1 else None
    api.attn_chunk(_dev(c.q), _dev(c.kb), _dev(c.vb), out, c.heads, c.n_kv, c.hd, c.pos0, c.tok, 2,
                   c.stride, pa, pm, splits, mode, ws)
    torch.cuda.synchronize()
    assert api.check_device_status() == 0
    ok, ma, rl = cases.attention_within_bar(want, out.cpu().numpy())
    assert ok, (ma, rl)


def test_chunk_2048_rows_at_6144_over_q4_sampled_rows():
    """The largest chunk of the 8192-token prefill over a q4 cache; every 97th query row is
    checked against the oracle over the dequantised values."""
    from hipml_b200 import api
    heads, n_kv, hd, pos0, tok, row = 24, 4, 256, 6144, 2048, 144
    stride = pos0 + tok
    g = torch.Generator(device="cuda").manual_seed(4)
    kf = torch.randn(stride, n_kv * hd, device="cuda", generator=g)
    vf = torch.randn(stride, n_kv * hd, device="cuda", generator=g)
    q = torch.randn(tok, heads * hd, device="cuda", generator=g)
    kc = torch.zeros(n_kv * stride * row, dtype=torch.uint8, device="cuda")
    vc = torch.zeros_like(kc)
    api.kv_encode_bulk(kf, vf, kc, vc, n_kv, hd, stride, 0, 0, stride, dtype=Q4)
    ws = torch.empty(api.attn_chunk_workspace_bytes(n_kv, hd, pos0, tok), dtype=torch.uint8,
                     device="cuda")
    out = torch.full((tok, heads * hd), float("nan"), device="cuda")
    api.attn_chunk(q, kc, vc, out, heads, n_kv, hd, pos0, tok, 2, stride, None, None, 1, 0, ws)
    torch.cuda.synchronize()
    assert api.check_device_status() == 0
    kq = cases.unpack_head_major(O.dequantize_q4(kc.cpu().numpy()), n_kv, stride, hd)
    vq = cases.unpack_head_major(O.dequantize_q4(vc.cpu().numpy()), n_kv, stride, hd)
    c = cases.ChunkCase(q.cpu().numpy(), kq, vq, None, None, heads, n_kv, hd, pos0, tok, stride)
    want = cases.chunk_expected(c, rows=(5, 97), threads=8)
    got = out.cpu().numpy()
    assert not np.isnan(got).any()
    ok, ma, rl = cases.attention_within_bar(want[5::97], got[5::97])
    assert ok, (ma, rl)


@pytest.mark.parametrize("seq", [1, 65, 700])
def test_decode_step_with_fused_append_equals_the_two_launches(seq):
    """hipml_attn_decode_kv_append over a q4_0 cache: row bytes and output identical to
    hipml_kv_encode + hipml_attn_decode_kv."""
    from hipml_b200 import api
    heads, n_kv, hd, scale, row = 24, 4, 256, 0.0625, 144
    stride = seq + 9
    rng = O.Rng(0xA994 + seq)
    q = rng.normals(heads * hd)
    k_row, v_row = rng.normals(n_kv * hd), rng.normals(n_kv * hd, 2.0)
    kc, vc = _poison_cache(n_kv, stride, hd), _poison_cache(n_kv, stride, hd)
    kc[:, :seq - 1] = O.quantize_q4(rng.normals(n_kv * (seq - 1) * hd)).reshape(n_kv, seq - 1, row)
    vc[:, :seq - 1] = O.quantize_q4(rng.normals(n_kv * (seq - 1) * hd)).reshape(n_kv, seq - 1, row)
    splits = api.decode_splits(seq)
    step = _step(seq - 1, seq)
    outs, caches = [], []
    for fused in (False, True):
        k, v = _dev(kc), _dev(vc)
        out = torch.full((heads * hd,), float("nan"), device="cuda")
        acc = torch.empty(heads * splits * hd, device="cuda")
        ml = torch.empty(heads * splits * 2, device="cuda")
        if fused:
            api.attn_decode_kv_append(step, _dev(k_row), _dev(v_row), _dev(q), k, v, acc, ml, out, heads,
                                      n_kv, hd, stride, scale, splits, selector=Q4)
        else:
            api.kv_encode(step, _dev(k_row), _dev(v_row), k, v, n_kv, hd, stride, dtype=Q4)
            api.attn_decode_kv(step, _dev(q), k, v, acc, ml, out, heads, n_kv, hd, stride, scale,
                               splits, selector=Q4)
        torch.cuda.synchronize()
        assert api.check_device_status() == 0
        outs.append(out)
        caches.append((k, v))
    assert torch.equal(caches[0][0], caches[1][0]) and torch.equal(caches[0][1], caches[1][1])
    assert torch.equal(outs[0], outs[1])
    kb = caches[1][0].cpu().numpy().reshape(n_kv, stride, row)
    vb = caches[1][1].cpu().numpy().reshape(n_kv, stride, row)
    _assert_close(O.attn_decode_kv(q, kb, vb, Q4, heads, n_kv, hd, seq, scale, stride=stride),
                  outs[1].cpu().numpy())
