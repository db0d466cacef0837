"""Attention front end and tail on the GPU against the CPU definition.

Cases follow the reference's parity table for these ops (crates/hipml-core/src/attn_parity.rs:
11-78: qg_split 6x64 seed 0x2222_3333_4444_5555, head_rmsnorm 6x64 with w = 1 + 0.1 N(0,1) seed
0x3333_4444_5555_6666, mrope 4x64 n_rot 64 sections 11/11/10/0 position 37 base 1e7 seed
0x4444_5555_6666_7777, q_gate 384 elements seed 0x5555_6666_7777_8888) and its norm + rope check
at position 37 (crates/hipml-cli/src/attn_cmd.rs:232-289, seed 0xF011_A77E_1234_5678), widened
to the shipped shape, a chunk at a non-zero position and the fused form with the q8_0 append.

Tolerances: the reference accepts abs 1e-4 OR rel 1e-3 for the norm and abs 1e-6 OR rel 1e-5 for
the rotation. Here the composite must stay within max-abs 5e-6 and relative-L2 1e-6 of the
oracle (the sum of squares is a tree instead of a chain, the rotation may contract to an FMA);
pure copies (split, gate rows) and cache bytes are bit-exact.
"""
import numpy as np
import pytest
import torch

import oracle as O

pytestmark = pytest.mark.gpu

SECTIONS = [11, 11, 10, 0]
THETA, EPS = 1e7, 1e-6
CANARY = 0xA5


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _ints(v):
    return torch.tensor(v, dtype=torch.int32, device="cuda")


def _assert_close(want, got, label=""):
    want, got = np.asarray(want, np.float32).ravel(), np.asarray(got, np.float32).ravel()
    ma, rl = O.max_abs(want, got), O.rel_l2(want, got)
    print(f"{label}: max_abs {ma:.2e} rel_l2 {rl:.2e}")
    assert np.all(np.isfinite(got))
    assert O.within(O.compare(want, got), O.TOL_DEFAULT)
    assert ma <= 5e-6 and rl <= 1e-6, (ma, rl)


def _front_inputs(seed, n_heads, n_kv, hd, tokens=1):
    rng = O.Rng(seed)
    qg = rng.normals(tokens * n_heads * 2 * hd).reshape(tokens, n_heads * 2 * hd)
    k = rng.normals(tokens * n_kv * hd).reshape(tokens, n_kv * hd)
    v = rng.normals(tokens * n_kv * hd, 1.5).reshape(tokens, n_kv * hd)
    qn = (1.0 + rng.normals(hd, 0.1)).astype(np.float32)
    kn = (1.0 + rng.normals(hd, 0.1)).astype(np.float32)
    return qg, k, v, qn, kn


@pytest.mark.parametrize("n_heads,n_kv,hd,n_rot,pos", [
    (6, 2, 64, 64, [37, 37, 37, 37]),      # the reference's op shapes, text position 37
    (4, 4, 64, 64, [37, 5, 9, 2]),         # distinct M-RoPE ids per section
    (24, 4, 256, 64, [1000, 1000, 1000, 1000]),   # the shipped shape
    (8, 2, 128, 32, [3, 3, 3, 3]),
])
def test_attn_front_one_token(n_heads, n_kv, hd, n_rot, pos):
    from hipml_b200 import api
    qg, k, _, qn, kn = _front_inputs(0xF011_A77E_1234_5678 + hd, n_heads, n_kv, hd)
    want_q, want_g, want_k = O.attn_front(qg[0], k[0], qn, kn, n_heads, n_kv, hd, n_rot, SECTIONS, pos,
                                          THETA, EPS)
    q = torch.full((n_heads * hd,), float("nan"), device="cuda")
    gate = torch.full((n_heads * hd,), float("nan"), device="cuda")
    dk = _dev(k[0])
    api.attn_front(_dev(qg[0]), q, gate, dk, _dev(qn), _dev(kn), n_heads, n_kv, hd, n_rot, SECTIONS,
                   _ints(pos), THETA, EPS)
    torch.cuda.synchronize()
    assert np.array_equal(gate.cpu().numpy(), want_g)
    _assert_close(want_q, q.cpu().numpy(), "front q")
    _assert_close(want_k, dk.cpu().numpy(), "front k")


def test_chunk_forms_at_a_non_zero_position():
    """qg_split_chunk + norm_rope_chunk over 37 tokens at position 29, token by token."""
    from hipml_b200 import api
    n_heads, n_kv, hd, n_rot, tokens, pos0 = 6, 2, 64, 64, 37, 29
    qg, k, _, qn, kn = _front_inputs(0x2222_3333_4444_5555, n_heads, n_kv, hd, tokens)
    q = torch.full((tokens, n_heads * hd), float("nan"), device="cuda")
    gate = torch.full((tokens, n_heads * hd), float("nan"), device="cuda")
    dk = _dev(k)
    api.qg_split_chunk(_dev(qg), q, gate, n_heads, hd, tokens)
    split = q.cpu().numpy().copy()
    api.norm_rope_chunk(q, dk, _dev(qn), _dev(kn), n_heads, n_kv, hd, n_rot, THETA, EPS, pos0, tokens)
    torch.cuda.synchronize()
    for t in range(tokens):
        wq, wg, wk = O.attn_front(qg[t], k[t], qn, kn, n_heads, n_kv, hd, n_rot, [0] * 4,
                                  [pos0 + t] * 4, THETA, EPS)
        assert np.array_equal(gate[t].cpu().numpy(), wg)
        assert np.array_equal(split[t], O.qg_split_f32(qg[t], n_heads, hd)[0])
        _assert_close(wq, q[t].cpu().numpy(), f"chunk q row {t}")
        _assert_close(wk, dk[t].cpu().numpy(), f"chunk k row {t}")


@pytest.mark.parametrize("n", [384, 383, 24 * 256 * 5])
def test_q_gate(n):
    from hipml_b200 import api
    rng = O.Rng(0x5555_6666_7777_8888)
    a, g = rng.normals(n, 0.5), rng.normals(n, 2.0)
    y = torch.full((n,), float("nan"), device="cuda")
    api.q_gate(_dev(a), _dev(g), y, n)
    want = O.q_gate_f32(a, g)
    got = y.cpu().numpy()
    assert O.within(O.compare(want, got), O.TOL_TIGHT)
    assert O.max_abs(want, got) <= 2e-7
    # in place, as the reference's chunk tail does (y aliases q)
    da = _dev(a)
    api.q_gate(da, _dev(g), da, n)
    assert np.array_equal(da.cpu().numpy(), got)


def _check_fused(tokens, pos0, stride, decode):
    from hipml_b200 import api
    n_heads, n_kv, hd, n_rot = 24, 4, 256, 64
    qg, k, v, qn, kn = _front_inputs(0xA77E_0001 + tokens, n_heads, n_kv, hd, tokens)
    q = torch.full((tokens, n_heads * hd), float("nan"), device="cuda")
    gate = torch.full((tokens, n_heads * hd), float("nan"), device="cuda")
    k_out = torch.full((tokens, n_kv * hd), float("nan"), device="cuda")
    kc = torch.full((n_kv * stride * 272,), CANARY, dtype=torch.uint8, device="cuda")
    vc = torch.full((n_kv * stride * 272,), CANARY, dtype=torch.uint8, device="cuda")
    if decode:
        pos = [pos0, pos0 + 3, pos0 + 7, pos0]
        api.attn_front_append_q8(_dev(qg), _dev(k), _dev(v), q, gate, _dev(qn), _dev(kn), kc, vc,
                                 n_heads, n_kv, hd, n_rot, THETA, EPS, tokens=1, stride=stride,
                                 sections=SECTIONS, pos=_ints(pos), step=_ints([pos0, pos0 + 1]),
                                 k_out=k_out)
    else:
        api.attn_front_append_q8(_dev(qg), _dev(k), _dev(v), q, gate, _dev(qn), _dev(kn), kc, vc,
                                 n_heads, n_kv, hd, n_rot, THETA, EPS, pos0=pos0, tokens=tokens,
                                 stride=stride, k_out=k_out)
    torch.cuda.synchronize()
    kb = kc.cpu().numpy().reshape(n_kv, stride, 272)
    vb = vc.cpu().numpy().reshape(n_kv, stride, 272)
    for t in range(tokens):
        p4 = pos if decode else [pos0 + t] * 4
        wq, wg, wk = O.attn_front(qg[t], k[t], qn, kn, n_heads, n_kv, hd, n_rot,
                                  SECTIONS if decode else [0] * 4, p4, THETA, EPS)
        assert np.array_equal(gate[t].cpu().numpy(), wg)
        _assert_close(wq, q[t].cpu().numpy(), f"fused q row {t}")
        got_k = k_out[t].cpu().numpy()
        _assert_close(wk, got_k, f"fused k row {t}")
        # cache rows: the q8_0 encode of exactly the rows the kernel produced / was given
        assert np.array_equal(kb[:, pos0 + t], O.quantize_q8(got_k).reshape(n_kv, 272))
        assert np.array_equal(vb[:, pos0 + t], O.quantize_q8(v[t]).reshape(n_kv, 272))
    # nothing else was written
    rest = np.ones(stride, dtype=bool)
    rest[pos0:pos0 + tokens] = False
    assert np.all(kb[:, rest] == CANARY) and np.all(vb[:, rest] == CANARY)


def test_fused_front_with_q8_append_chunk():
    _check_fused(tokens=50, pos0=131, stride=300, decode=False)


def test_fused_front_with_q8_append_one_decode_token():
    _check_fused(tokens=1, pos0=37, stride=64, decode=True)


def test_fused_front_without_caches_and_argument_errors():
    from hipml_b200 import api
    n_heads, n_kv, hd = 24, 4, 256
    qg, k, v, qn, kn = _front_inputs(9, n_heads, n_kv, hd, 3)
    q = torch.empty(3, n_heads * hd, device="cuda")
    gate = torch.empty(3, n_heads * hd, device="cuda")
    api.attn_front_append_q8(_dev(qg), _dev(k), _dev(v), q, gate, _dev(qn), _dev(kn), None, None,
                             n_heads, n_kv, hd, 64, THETA, EPS, pos0=5, tokens=3)
    wq, _, _ = O.attn_front(qg[2], k[2], qn, kn, n_heads, n_kv, hd, 64, [0] * 4, [7] * 4, THETA, EPS)
    _assert_close(wq, q[2].cpu().numpy(), "no-cache q")
    z = torch.zeros(16, device="cuda")
    with pytest.raises(Exception, match="head_dim 256"):
        api.attn_front_append_q8(z, z, z, z, z, z, z, None, None, 2, 1, 64, 64, THETA, EPS)
    with pytest.raises(Exception, match="beyond KV cache"):
        c = torch.zeros(272 * 4 * 4, dtype=torch.uint8, device="cuda")
        api.attn_front_append_q8(_dev(qg), _dev(k), _dev(v), q, gate, _dev(qn), _dev(kn), c, c,
                                 n_heads, n_kv, hd, 64, THETA, EPS, pos0=3, tokens=3, stride=4)


def test_gated_decode_equals_decode_then_gate():
    """The output gate fused into the decode fold: attention over a q8_0 cache of 700 rows, then
    * sigmoid(gate), against the oracle's attention followed by its q_gate."""
    from hipml_b200 import api
    heads, n_kv, hd, seq, scale = 24, 4, 256, 700, 0.0625
    rng = O.Rng(0x6A7E)
    q = rng.normals(heads * hd)
    gate = rng.normals(heads * hd, 2.0)
    kb = O.quantize_q8(rng.normals(n_kv * seq * hd)).reshape(n_kv, seq, 272)
    vb = O.quantize_q8(rng.normals(n_kv * seq * hd)).reshape(n_kv, seq, 272)
    want = O.q_gate_f32(O.attn_decode_kv_q8(q, kb, vb, heads, n_kv, hd, seq, scale), gate)
    splits = api.decode_splits(seq)
    out = torch.full((heads * hd,), float("nan"), device="cuda")
    acc = torch.full((heads * splits * hd,), float("nan"), device="cuda")
    ml = torch.full((heads * splits * 2,), float("nan"), device="cuda")
    step = _ints([seq - 1, seq, 0, 0, 0, 0, 0, 0])
    api.attn_decode_kv_gated(step, _dev(q), _dev(kb), _dev(vb), acc, ml, out, _dev(gate), heads, n_kv,
                             hd, seq, scale, splits)
    got = out.cpu().numpy()
    assert O.max_abs(want, got) <= 2e-6 and O.rel_l2(want, got) <= 1e-5


@pytest.mark.parametrize("splits", [1, 3])
def test_gated_chunk_attention_equals_chunk_then_gate(splits):
    """The gate fused into the chunk attention's epilogue (one pass) and into the combine pass
    (key slices): bit-identical to the ungated call followed by q_gate on the same rows."""
    from hipml_b200 import api
    heads, n_kv, hd, tok, pos0, stride = 24, 4, 256, 45, 260, 320
    g = torch.Generator(device="cuda").manual_seed(11)
    q = torch.randn(tok, heads * hd, device="cuda", generator=g)
    gate = 2.0 * torch.randn(tok, heads * hd, device="cuda", generator=g)
    kf = torch.randn(pos0 + tok, n_kv * hd, device="cuda", generator=g)
    vf = torch.randn(pos0 + tok, n_kv * hd, device="cuda", generator=g)
    kc = torch.zeros(n_kv * stride * 272, dtype=torch.uint8, device="cuda")
    vc = torch.zeros_like(kc)
    api.kv_encode_bulk(kf, vf, kc, vc, n_kv, hd, stride, 0, 0, pos0 + tok)
    cap = 384
    ws = torch.empty(api.attn_chunk_workspace_bytes(n_kv, hd, 0, cap), dtype=torch.uint8, device="cuda")
    api.attn_chunk_stage(kc, vc, n_kv, hd, 1, stride, 0, pos0 + tok, cap, ws)
    qslots = (tok + 31) // 32 * 32
    pa = torch.empty(splits * qslots * heads * hd, device="cuda") if splits > 1 else None
    pm = torch.empty(splits * qslots * heads * 2, device="cuda") if splits > 1 else None
    plain = torch.full((tok, heads * hd), float("nan"), device="cuda")
    gated = torch.full((tok, heads * hd), float("nan"), device="cuda")
    api.attn_chunk_staged(q, plain, heads, n_kv, hd, pos0, tok, cap, ws, pa, pm, splits)
    api.attn_chunk_staged_gated(q, gated, gate, heads, n_kv, hd, pos0, tok, cap, ws, pa, pm, splits)
    assert api.check_device_status() == 0
    want = O.q_gate_f32(plain.cpu().numpy().ravel(), gate.cpu().numpy().ravel())
    got = gated.cpu().numpy().ravel()
    assert np.all(np.isfinite(got))
    assert O.max_abs(want, got) <= 5e-7
