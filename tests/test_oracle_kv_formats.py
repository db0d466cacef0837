"""The oracle against the reference's own KV-format tests.

Each test restates one test of crates/hipml-core/tests/kv_formats.rs (the
known-answer vectors, the bit layout and the error bounds) so the C
restatement of kv.rs / rng.rs / ops.rs is pinned on the reference's fixtures.
"""
import numpy as np

import oracle as O


def test_block_byte_counts_are_the_documented_layout():
    # kv_formats.rs:16-22: 2 (K,V) * 4 kv heads * 16 layers * 256/32 blocks * 34 B
    assert O.Q8_BLOCK_BYTES == 34
    row_bytes = 256 // O.BLOCK * O.Q8_BLOCK_BYTES
    assert row_bytes == 272
    assert 2 * 4 * 16 * row_bytes == 34_816


def test_f16_round_trips_exactly_and_rounds_to_nearest():
    # kv_formats.rs:25-40
    for h in [0x0000, 0x3800, 0x3C00, 0xBC00, 0x7BFF, 0x0001, 0x03FF, 0x7C00]:
        f = O.f16_to_f32(h)
        if h & 0x7FFF == 0x7C00:
            continue
        assert O.f32_to_f16(f) == h, f"f16 {h:#06x} did not round trip"
    assert np.float32(O.f16_to_f32(O.f32_to_f16(0.1))) == np.float32(0.099_975_586)
    assert O.f32_to_f16(float("inf")) == 0x7C00
    assert O.f32_to_f16(-0.0) == 0x8000


def test_f16_conversion_agrees_with_ieee_half_everywhere():
    # Not in the reference: every f16 bit pattern decodes like IEEE binary16 and
    # a dense sweep of f32 values rounds like numpy's round-to-nearest-even.
    hs = np.arange(0x10000, dtype=np.uint16)
    want = hs.view(np.float16).astype(np.float32)
    got = np.array([O.f16_to_f32(int(h)) for h in hs], dtype=np.float32)
    finite = np.isfinite(want)
    assert np.array_equal(got[finite], want[finite])
    assert np.all(np.isnan(got[np.isnan(want)]))
    rng = np.random.default_rng(5)
    xs = np.concatenate([
        rng.standard_normal(20000).astype(np.float32) * 10.0 ** rng.integers(-9, 6, 20000),
        np.array([65504.0, 65519.9, 65520.0, 1e9, 5.96e-8, 2.98e-8, 2.99e-8, 6.1e-5, 0.0],
                 dtype=np.float32),
    ]).astype(np.float32)
    with np.errstate(over="ignore"):
        want16 = xs.astype(np.float16).view(np.uint16)
    got16 = np.array([O.f32_to_f16(float(x)) for x in xs], dtype=np.uint16)
    assert np.array_equal(got16, want16)


def test_q8_known_vector_is_exact_and_packs_as_documented():
    # kv_formats.rs:43-61: amax 63.5 -> d = 0.5, exact in f16
    xs = np.zeros(32, dtype=np.float32)
    xs[0], xs[1] = 63.5, -63.5
    for j in range(2, 32):
        xs[j] = 0.5 * (j - 8.0)
    b = O.quantize_q8(xs)
    assert b.size == 34
    assert list(b[0:2]) == [0x00, 0x38], "scale must be f16 0.5"
    assert b[2] == 127
    assert b[3] == np.uint8(np.int8(-127))
    back = O.dequantize_q8(b)
    assert np.array_equal(back, xs)


def test_q8_round_trip_error_is_half_a_step():
    # kv_formats.rs:64-89
    rng = O.Rng(0x08)
    for _ in range(64):
        xs = rng.normals(32, 3.0)
        step = np.float32(np.max(np.abs(xs))) / np.float32(127.0)
        back = O.dequantize_q8(O.quantize_q8(xs))
        err = np.max(np.abs(xs - back))
        assert err <= step * 0.5625 + 1e-6
        assert np.all((back == 0.0) | (np.sign(xs) == np.sign(back)))
    zeros = O.quantize_q8(np.zeros(32, dtype=np.float32))
    assert list(zeros[0:2]) == [0, 0]
    assert np.all(O.dequantize_q8(zeros) == 0.0)


def test_row_layout_matches_block_order():
    # kv_formats.rs:140-162 (restated for q8): value (h, pos, d) comes back from
    # block ((h*seq + pos)*nb + d/32), element d%32.
    n_kv, seq, dim = 2, 7, 64
    rng = O.Rng(77)
    values = rng.normals(n_kv * seq * dim, 0.7)
    b = O.quantize_q8(values)
    nb, bb = dim // 32, 34
    back = O.dequantize_q8(b)
    for h in range(n_kv):
        for pos in range(seq):
            for d in range(dim):
                at = ((h * seq + pos) * nb + d // 32) * bb
                want = O.dequantize_q8(b[at:at + bb])[d % 32]
                assert back[(h * seq + pos) * dim + d] == want


def test_quantized_attention_equals_attention_over_decoded_values():
    # kv_formats.rs:165-195 (Q8 arm; seed 0xABCD + dtype id 0)
    heads, n_kv, dim, seq = 6, 1, 64, 257
    rng = O.Rng(0xABCD)
    q = rng.normals(heads * dim)
    k = rng.normals(n_kv * seq * dim, 0.3)
    v = rng.normals(n_kv * seq * dim)
    kb, vb = O.quantize_q8(k), O.quantize_q8(v)
    quantized = O.attn_decode_kv_q8(q, kb, vb, heads, n_kv, dim, seq, 0.125)
    dense = O.attn_decode_f32(q, O.dequantize_q8(kb), O.dequantize_q8(vb), heads, n_kv, dim, seq,
                              0.125)
    assert np.max(np.abs(quantized - dense)) < 1e-5


def test_quantized_attention_error_against_the_f32_cache_is_small():
    # kv_formats.rs:198-227 (Q8 bound 2e-3)
    heads, n_kv, dim, seq = 6, 1, 64, 512
    rng = O.Rng(0xFEED)
    q = rng.normals(heads * dim)
    k = rng.normals(n_kv * seq * dim, 0.3)
    v = rng.normals(n_kv * seq * dim)
    exact = O.attn_decode_f32(q, k, v, heads, n_kv, dim, seq, 0.125)
    got = O.attn_decode_kv_q8(q, O.quantize_q8(k), O.quantize_q8(v), heads, n_kv, dim, seq, 0.125)
    assert np.max(np.abs(exact - got)) <= 2e-3


def test_synthetic_bench_cache_is_well_formed():
    # kv_formats.rs:230-246
    b = O.synthetic_blocks_q8(1000, 7)
    assert b.size == 1000 * 34
    back = O.dequantize_q8(b)
    assert np.all(np.isfinite(back)) and np.any(np.abs(back) > 0)
    for i in range(1000):
        d = O.f16_to_f32(int(b[i * 34]) | (int(b[i * 34 + 1]) << 8))
        assert 0.01 <= d < 0.05, f"scale {d} out of range"


def test_rng_matches_an_independent_numpy_restatement():
    # rng.rs:13-49 restated with Python integers and numpy float32, so the C
    # generator is checked against a second, independent implementation.
    def ref_stream(seed, n):
        mask = (1 << 64) - 1
        s = (seed | 1) & mask
        out = []
        for _ in range(n):
            s ^= s >> 12
            s ^= (s << 25) & mask
            s ^= s >> 27
            out.append((s * 0x2545F4914F6CDD1D) & mask)
        return out

    for seed in [0, 1, 0x9E00_0001, 0xDDDD_EEEE_FFFF_0003]:
        rng = O.Rng(seed)
        raw = ref_stream(seed, 16)
        assert [rng.next_u64() for _ in range(16)] == raw
        rng = O.Rng(seed)
        un = np.array([(r >> 40) for r in raw], dtype=np.float32) / np.float32(1 << 24)
        got_u = np.array([rng.uniform() for _ in range(16)], dtype=np.float32)
        assert np.array_equal(got_u, un)
        rng = O.Rng(seed)
        normals = rng.normals(8)
        u1 = np.maximum(un[0::2], np.float32(1e-7))
        u2 = un[1::2]
        want = np.sqrt(np.float32(-2.0) * np.log(u1)) * np.cos(np.float32(6.2831855) * u2)
        # numpy's float32 log/cos may differ from libm in the last bit
        assert np.allclose(normals, want.astype(np.float32), rtol=2e-6, atol=1e-7)
    first = O.Rng(0).normals(4)
    assert np.allclose(first, [-0.75778687, -0.26419523, 0.49144033, -0.29645920], atol=2e-7)
