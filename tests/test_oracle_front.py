"""The oracle's attention front end and tail against the reference's own CPU checks.

crates/hipml-core/tests/forward_ops.rs:19-47 (rope_multi: full rotation is plain NeoX; only the
first n_rot channels rotate; pair k has frequency base^(-2k/n_rot), hand-computed values) and
the definitions of crates/hipml-core/src/ops.rs:181-187, 315-329, 354-360 restated in numpy.
"""
import numpy as np

import oracle as O


def _close(a, b, tol):
    return abs(a - b) <= tol * (1.0 + max(abs(a), abs(b)))


def test_rope_multi_with_full_rotation_is_plain_neox():
    x = (np.arange(8) * 0.5 - 1.0).astype(np.float32)
    multi = O.rope_multi_f32(x, 1, 8, 8, [0] * 4, [3] * 4, 10_000.0)
    neox = O.rope_neox_f32(x, 1, 8, 3, 10_000.0)
    assert all(_close(a, b, 1e-5) for a, b in zip(multi, neox))


def test_rope_multi_rotates_only_the_first_n_rot_channels():
    x = (np.arange(8) + 1.0).astype(np.float32)
    y = O.rope_multi_f32(x, 1, 8, 4, [0] * 4, [5] * 4, 10_000.0)
    assert np.array_equal(y[4:], x[4:])
    assert abs(y[0] - x[0]) > 1e-3 and abs(y[2] - x[2]) > 1e-3
    expect0 = x[0] * np.cos(np.float32(5.0)) - x[2] * np.sin(np.float32(5.0))
    assert _close(y[0], expect0, 1e-5)
    ang = 5.0 * 10_000.0 ** (-2.0 / 4.0)
    expect1 = x[1] * np.float32(np.cos(ang)) - x[3] * np.float32(np.sin(ang))
    assert _close(y[1], expect1, 1e-5)


def test_rope_sections_pick_the_position_id():
    """Pair k uses id 0 for k % 32 < 11, id 1 for < 22, id 2 for < 32 (sections 11/11/10/0)."""
    rng = O.Rng(0x4444_5555_6666_7777)
    x = rng.normals(4 * 64)
    pos = [37, 5, 9, 2]
    y = O.rope_multi_f32(x, 4, 64, 64, [11, 11, 10, 0], pos, 1e7)
    xs, ys = x.reshape(4, 64), y.reshape(4, 64)
    for k in range(32):
        p = pos[0] if k < 11 else pos[1] if k < 22 else pos[2]
        ang = p * (1e7 ** (-2.0 * k / 64.0))
        cs, sn = np.float32(np.cos(ang)), np.float32(np.sin(ang))
        want = xs[:, k] * cs - xs[:, k + 32] * sn
        assert np.allclose(ys[:, k], want, rtol=0, atol=2e-6)
    # text: the same id four times is plain rope over n_rot channels
    same = O.rope_multi_f32(x, 4, 64, 64, [11, 11, 10, 0], [37] * 4, 1e7)
    plain = O.rope_multi_f32(x, 4, 64, 64, [0] * 4, [37] * 4, 1e7)
    assert np.array_equal(same, plain)


def test_head_rmsnorm_is_the_f32_definition():
    rng = O.Rng(0x3333_4444_5555_6666)
    x = rng.normals(6 * 64)
    w = (1.0 + rng.normals(64, 0.1)).astype(np.float32)
    got = O.head_rmsnorm_f32(x, w, 6, 64, 1e-6).reshape(6, 64)
    for h, row in enumerate(x.reshape(6, 64)):
        s = np.float32(0)
        for v in row:
            s = np.float32(s + np.float32(v * v))
        scale = np.float32(1.0) / np.sqrt(np.float32(s / np.float32(64) + np.float32(1e-6)))
        assert np.array_equal(got[h], (row * scale * w).astype(np.float32))


def test_qg_split_and_q_gate():
    rng = O.Rng(0x2222_3333_4444_5555)
    qg = rng.normals(6 * 128)
    q, gate = O.qg_split_f32(qg, 6, 64)
    v = qg.reshape(6, 2, 64)
    assert np.array_equal(q.reshape(6, 64), v[:, 0]) and np.array_equal(gate.reshape(6, 64), v[:, 1])
    rng = O.Rng(0x5555_6666_7777_8888)
    a, g = rng.normals(384, 0.5), rng.normals(384, 2.0)
    y = O.q_gate_f32(a, g)
    want = a.astype(np.float64) / (1.0 + np.exp(-g.astype(np.float64)))
    assert np.abs(y - want).max() < 1e-6
    assert O.q_gate_f32(np.float32([3.0]), np.float32([0.0]))[0] == np.float32(1.5)
