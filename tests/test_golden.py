"""The oracle against the committed golden vectors (tests/golden/make_golden.py)."""
import os

import numpy as np

import oracle as O
from tests import cases
from tests.golden.make_golden import CHUNK_ROWS

GOLDEN = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden",
                              "attention_golden.npz"))


def test_q8_known_vector_bytes_are_the_references():
    b = GOLDEN["q8_known_vector_bytes"]
    assert list(b[0:4]) == [0x00, 0x38, 127, 129]  # scale f16 0.5, codes +127, -127
    xs = np.zeros(32, dtype=np.float32)
    xs[0], xs[1] = 63.5, -63.5
    xs[2:] = 0.5 * (np.arange(2, 32, dtype=np.float32) - 8.0)
    assert np.array_equal(O.quantize_q8(xs), b)


def test_kv_encode_case_bytes():
    k, v = cases.kv_encode_case_inputs()
    c = cases.KV_ENCODE_CASE
    krows, vrows = cases.kv_encode_expected_bytes(k, v, c["n_kv"], c["head_dim"])
    assert np.array_equal(np.concatenate(krows), GOLDEN["kv_encode_q8_k_bytes"])
    assert np.array_equal(np.concatenate(vrows), GOLDEN["kv_encode_q8_v_bytes"])


def test_decode_cases_reproduce():
    for c in cases.KV_CASES:
        if c.seq > 1000:
            continue  # the 4096-row case is covered on the GPU side; keep the CPU suite short
        q, kb, vb = cases.kv_case_inputs(c)
        got = cases.kv_case_expected(c, q, kb, vb)
        assert O.within(O.compare(GOLDEN[c.name], got), O.TOL_TIGHT), c.name
    assert O.within(O.compare(GOLDEN["decode_pm_f32"], cases.decode_f32_case()["expected"]),
                    O.TOL_TIGHT)


def test_chunk_cases_reproduce():
    f32 = cases.chunk_expected(cases.chunk_case_f32())[list(CHUNK_ROWS)]
    q8 = cases.chunk_expected(cases.chunk_case_q8())[list(CHUNK_ROWS)]
    assert O.within(O.compare(GOLDEN["chunk_f32_37_at_29_rows"], f32), O.TOL_TIGHT)
    assert O.within(O.compare(GOLDEN["chunk_q8_37_at_29_rows"], q8), O.TOL_TIGHT)
