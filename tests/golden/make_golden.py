"""Writes tests/golden/attention_golden.npz: oracle outputs for the reference's seeded
parity cases (inputs are regenerated from the seeds, so only outputs are stored).

The reference is Rust and cannot be built or imported where this runs, so these vectors come
from the C restatement in oracle/ (itself pinned on the reference's known-answer tests, see
tests/test_oracle_kv_formats.py). They freeze the oracle against drift and give the GPU
tests a fixed target that does not depend on the host's libm at test time.

Run from the repository root:  python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

import oracle as O  # noqa: E402
from tests import cases  # noqa: E402

CHUNK_ROWS = (0, 18, 36)


def main():
    out = {}
    for c in cases.KV_CASES:
        q, kb, vb = cases.kv_case_inputs(c)
        out[c.name] = cases.kv_case_expected(c, q, kb, vb)
    k, v = cases.kv_encode_case_inputs()
    krows, vrows = cases.kv_encode_expected_bytes(k, v, cases.KV_ENCODE_CASE["n_kv"],
                                                  cases.KV_ENCODE_CASE["head_dim"])
    out["kv_encode_q8_k_bytes"] = np.concatenate(krows)
    out["kv_encode_q8_v_bytes"] = np.concatenate(vrows)
    out["chunk_f32_37_at_29_rows"] = cases.chunk_expected(cases.chunk_case_f32())[list(CHUNK_ROWS)]
    out["chunk_q8_37_at_29_rows"] = cases.chunk_expected(cases.chunk_case_q8())[list(CHUNK_ROWS)]
    out["decode_pm_f32"] = cases.decode_f32_case()["expected"]
    # the reference's own known-answer vector for the format (tests/kv_formats.rs:43-61)
    xs = np.zeros(32, dtype=np.float32)
    xs[0], xs[1] = 63.5, -63.5
    xs[2:] = 0.5 * (np.arange(2, 32, dtype=np.float32) - 8.0)
    out["q8_known_vector_bytes"] = O.quantize_q8(xs)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "attention_golden.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
