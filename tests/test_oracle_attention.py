"""The oracle's attention against the reference's identity tests.

Restates crates/hipml-core/tests/parity_reference.rs:222-302 (the reference
stores no golden output tensors for attention; its CPU tests are identities
that hold by construction), plus cross-checks between the three CPU attention
functions the reference defines.
"""
import math

import numpy as np

import oracle as O


def test_attention_matches_a_hand_computed_case():
    # parity_reference.rs:222-233
    out = O.attn_decode_f32([1.0, 0.0], [1.0, 0.0, 0.0, 1.0], [10.0, 0.0, 0.0, 100.0],
                            1, 1, 2, 2, 1.0)
    e = math.e
    p0, p1 = e / (e + 1.0), 1.0 / (e + 1.0)
    assert abs(out[0] - p0 * 10.0) < 1e-5
    assert abs(out[1] - p1 * 100.0) < 1e-5


def test_attention_of_uniform_scores_is_the_mean_of_values():
    # parity_reference.rs:236-254
    heads, kv, dim, seq = 4, 1, 8, 16
    q = np.zeros(heads * dim, dtype=np.float32)
    k = np.ones(kv * seq * dim, dtype=np.float32)
    v = O.Rng(29).normals(kv * seq * dim)
    out = O.attn_decode_f32(q, k, v, heads, kv, dim, seq, 0.1).reshape(heads, dim)
    mean = v.reshape(seq, dim).sum(axis=0) / seq
    assert np.max(np.abs(out - mean[None, :])) < 1e-5


def test_attention_routes_each_query_head_to_its_kv_head():
    # parity_reference.rs:257-276
    heads, kv, dim, seq = 4, 2, 4, 3
    q = np.ones(heads * dim, dtype=np.float32)
    k = np.ones(kv * seq * dim, dtype=np.float32)
    v = np.concatenate([np.full(seq * dim, 1.0), np.full(seq * dim, 7.0)]).astype(np.float32)
    out = O.attn_decode_f32(q, k, v, heads, kv, dim, seq, 0.1).reshape(heads, dim)
    assert np.max(np.abs(out[:2] - 1.0)) < 1e-5
    assert np.max(np.abs(out[2:] - 7.0)) < 1e-5


def test_attention_output_is_a_convex_combination():
    # parity_reference.rs:279-302
    heads, kv, dim, seq = 2, 1, 6, 32
    rng = O.Rng(31)
    q = rng.normals(heads * dim)
    k = rng.normals(kv * seq * dim)
    v = rng.normals(kv * seq * dim)
    out = O.attn_decode_f32(q, k, v, heads, kv, dim, seq, 0.125).reshape(heads, dim)
    vv = v.reshape(seq, dim)
    assert np.all(out >= vv.min(axis=0) - 1e-5) and np.all(out <= vv.max(axis=0) + 1e-5)


def test_position_major_and_head_major_f32_attention_agree():
    # attention.rs:56-102 (position-major cache) and ops.rs:530-588 (kv-major
    # cache) are the same arithmetic in the same order: bit-identical outputs.
    heads, kv, dim, seq = 6, 2, 32, 19
    rng = O.Rng(41)
    q = rng.normals(heads * dim)
    k = rng.normals(seq * kv * dim).reshape(seq, kv, dim)
    v = rng.normals(seq * kv * dim).reshape(seq, kv, dim)
    a = O.attn_causal_f32(q, k, v, heads, kv, dim, seq, 0.2)
    b = O.attn_decode_f32(q, k.transpose(1, 0, 2), v.transpose(1, 0, 2), heads, kv, dim, seq, 0.2)
    assert np.array_equal(a, b)


def test_chunk_rows_are_causal_and_thread_count_does_not_change_them():
    heads, kv, dim, pos0, tok = 4, 2, 32, 5, 9
    rng = O.Rng(43)
    q = rng.normals(tok * heads * dim).reshape(tok, heads * dim)
    k = rng.normals((pos0 + tok) * kv * dim)
    v = rng.normals((pos0 + tok) * kv * dim)
    one = O.attn_chunk_f32(q, k, v, heads, kv, dim, pos0, tok, 0.25)
    many = O.attn_chunk_f32(q, k, v, heads, kv, dim, pos0, tok, 0.25, threads=4)
    assert np.array_equal(one, many)
    for t in range(tok):
        row = O.attn_causal_f32(q[t], k, v, heads, kv, dim, pos0 + t + 1, 0.25)
        assert np.array_equal(one[t], row)
    # a future key must not change an earlier row
    k2 = k.copy()
    k2[(pos0 + tok - 1) * kv * dim:] += 3.0
    again = O.attn_chunk_f32(q, k2, v, heads, kv, dim, pos0, tok, 0.25)
    assert np.array_equal(again[: tok - 1], one[: tok - 1])
    assert not np.array_equal(again[tok - 1], one[tok - 1])
    sampled = O.attn_chunk_f32(q, k, v, heads, kv, dim, pos0, tok, 0.25, row0=1, row_step=3)
    assert np.array_equal(sampled[1::3], one[1::3]) and np.all(np.isnan(sampled[0]))


def test_strided_decode_reads_only_live_rows():
    heads, kv, dim, seq, stride = 6, 2, 64, 11, 17
    rng = O.Rng(47)
    q = rng.normals(heads * dim)
    row = dim // 32 * 34
    k = O.quantize_q8(rng.normals(kv * seq * dim, 0.3)).reshape(kv, seq, row)
    v = O.quantize_q8(rng.normals(kv * seq * dim)).reshape(kv, seq, row)
    dense = O.attn_decode_kv_q8(q, k, v, heads, kv, dim, seq, 0.125)
    pad_k = np.full((kv, stride, row), 0xFF, dtype=np.uint8)
    pad_v = np.full((kv, stride, row), 0xFF, dtype=np.uint8)
    pad_k[:, :seq], pad_v[:, :seq] = k, v
    strided = O.attn_decode_kv_q8(q, pad_k, pad_v, heads, kv, dim, seq, 0.125, stride=stride)
    assert np.array_equal(dense, strided)


def test_compare_and_tolerance_rule():
    # parity.rs:50-53,58-80; parity_reference.rs:215-219
    st = O.compare([1.0, 2.0], [1.0, 2.0001])
    assert O.within(st, (1e-3, 1e-3))
    st = O.compare([1.0, 2.0], [1.0, 3.0])
    assert not O.within(st, (1e-3, 1e-3)) and st[0] > 0.9
    # OR rule: a large relative error on a tiny value still passes on abs
    st = O.compare([1e-9], [2e-9])
    assert O.within(st, O.TOL_DEFAULT)
