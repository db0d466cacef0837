"""The oracle's q4_0 format against the reference's own format tests
(crates/hipml-core/tests/kv_formats.rs:92-137 and the row-layout law of :139-160)."""
import numpy as np

import oracle as O


def test_q4_known_vector_packs_low_nibble_j_high_nibble_j16():
    xs = np.array([0.25 * ((j % 16) - 8.0) for j in range(32)], dtype=np.float32)
    b = O.quantize_q4(xs)
    assert b.size == 18
    assert list(b[:2]) == [0x00, 0x34]                     # f16 0.25
    assert [int(v) for v in b[2:]] == [(j << 4) | j for j in range(16)]
    assert np.array_equal(O.dequantize_q4(b), xs)


def test_q4_extreme_maps_exactly_and_error_is_bounded():
    for vmax in (2.0, -2.0, 0.125, -0.125):
        xs = np.full(32, 0.1, dtype=np.float32)
        xs[5] = vmax
        assert O.dequantize_q4(O.quantize_q4(xs))[5] == np.float32(vmax)
    rng = O.Rng(0x4_0)
    for _ in range(64):
        xs = rng.normals(32, 2.0)
        back = O.dequantize_q4(O.quantize_q4(xs))
        assert np.abs(xs - back).max() <= np.abs(xs).max() / 8.0 + 1e-6


def test_q4_edge_values():
    z = O.quantize_q4(np.zeros(32, dtype=np.float32))
    # vmax = 0 gives d = -0.0 (f16 0x8000), every nibble 8
    assert list(z[:2]) == [0x00, 0x80] and np.all(z[2:] == 0x88)
    assert np.all(O.dequantize_q4(z) == 0.0)
    xs = np.full(32, 1.0, dtype=np.float32)
    xs[3] = np.nan                                            # a NaN encodes as nibble 0
    b = O.quantize_q4(xs)
    assert (b[2 + 3] & 0x0F) == 0
    # ties on |v|: the first element decides the sign of the scale
    xs = np.zeros(32, dtype=np.float32)
    xs[2], xs[9] = 3.0, -3.0
    d = O.f16_to_f32(int(O.quantize_q4(xs)[0]) | (int(O.quantize_q4(xs)[1]) << 8))
    assert d == np.float32(-3.0 / 8.0)


def test_q4_rows_and_decode_agree_with_dequantised_attention():
    """A q4 row of head_dim 256 is 8 blocks = 144 bytes; the decode over the bytes equals the
    f32 decode over the dequantised values."""
    heads, n_kv, hd, seq = 8, 2, 64, 37
    rng = O.Rng(0x9E00_000B)
    q = rng.normals(heads * hd)
    kb = O.quantize_q4(rng.normals(n_kv * seq * hd, 0.3))
    vb = O.quantize_q4(rng.normals(n_kv * seq * hd))
    assert O.quantize_q4(np.zeros(256, np.float32)).size == 144
    got = O.attn_decode_kv(q, kb, vb, 1, heads, n_kv, hd, seq, 0.125)
    want = O.attn_decode_f32(q, O.dequantize_q4(kb), O.dequantize_q4(vb), heads, n_kv, hd, seq, 0.125)
    assert O.max_abs(want, got) <= 1e-6
    s = O.synthetic_blocks_q4(100, 7).reshape(100, 18)
    d = np.array([O.f16_to_f32(int(r[0]) | (int(r[1]) << 8)) for r in s])
    assert np.all(d >= 0.0099) and np.all(d < 0.0501)
