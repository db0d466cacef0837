"""The callers either side of the attention kernels that only move pointers and positions:
verify columns over a shared cache, a row block of several slots' tails, and the attention
half of a prefix snapshot.

Reference: crates/hipml-model/src/gpu/attn_tile.rs:225-295 (deep_attention_cols: every column's
partials are the ones its one-column launch writes), crates/hipml-kernels/src/attn_gpu/imp/
attn_rows.rs:1-203 with crates/hipml-model/src/gpu/batch/rows.rs:320-360 (a tail's KV and
outputs are unchanged by being batched with other tails), crates/hipml-model/src/gpu/prefix.rs:
30-43 (the quantised snapshot is a copy of the head-major rows).
"""
import numpy as np
import pytest
import torch

import oracle as O
from tests import cases

pytestmark = pytest.mark.gpu

H, KV, D, ROW, SCALE = 24, 4, 256, 272, 0.0625


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _ints(v):
    return torch.tensor(v, dtype=torch.int32, device="cuda")


def _filled_cache(rng, stride, rows):
    """A q8_0 cache pair with `rows` live rows of N(0,1) data and canary bytes behind them."""
    kb = np.full((KV, stride, ROW), 0xA5, dtype=np.uint8)
    vb = np.full((KV, stride, ROW), 0xA5, dtype=np.uint8)
    if rows:
        kb[:, :rows] = O.quantize_q8(rng.normals(KV * rows * D)).reshape(KV, rows, ROW)
        vb[:, :rows] = O.quantize_q8(rng.normals(KV * rows * D)).reshape(KV, rows, ROW)
    return kb, vb


@pytest.mark.parametrize("pos0,cols", [(200, 5), (0, 3), (1023, 2)])
def test_verify_columns_are_bit_identical_to_one_column_launches(pos0, cols):
    from hipml_b200 import api
    stride = pos0 + cols + 11
    rng = O.Rng(0xC015 + pos0)
    kb, vb = _filled_cache(rng, stride, pos0 + cols)   # the verify step appended all columns' rows
    q = rng.normals(cols * H * D).reshape(cols, H * D)
    dk, dv, dq = _dev(kb), _dev(vb), _dev(q)
    # the reference groups columns of equal split count; these shapes give one group
    splits = api.decode_splits(pos0 + 1)
    assert all(api.decode_splits(pos0 + c + 1) == splits for c in range(cols))
    acc_slot, ml_slot, q_slot = H * splits * D, H * splits * 2, H * D
    pos = _ints([[pos0 + c, pos0 + c + 1] for c in range(cols)])
    acc = torch.full((cols * acc_slot,), float("nan"), device="cuda")
    ml = torch.full((cols * ml_slot,), float("nan"), device="cuda")
    out = torch.full((cols, H * D), float("nan"), device="cuda")
    api.attn_decode_cols(pos, dq, dk, dv, acc, ml, out, H, KV, D, stride, SCALE, splits, cols,
                         acc_slot, ml_slot, q_slot)
    got = out.cpu().numpy()
    for c in range(cols):
        seq = pos0 + c + 1
        one = torch.full((H * D,), float("nan"), device="cuda")
        a1 = torch.full((acc_slot,), float("nan"), device="cuda")
        m1 = torch.full((ml_slot,), float("nan"), device="cuda")
        api.attn_decode_kv(_ints([seq - 1, seq, 0, 0, 0, 0, 0, 0]), dq[c], dk, dv, a1, m1, one, H, KV,
                           D, stride, SCALE, splits)
        assert np.array_equal(one.cpu().numpy(), got[c]), f"column {c} differs from its own launch"
        want = O.attn_decode_kv_q8(q[c], kb, vb, H, KV, D, seq, SCALE, stride=stride)
        ok, ma, rl = cases.attention_within_bar(want, got[c])
        assert ok and ma <= 2e-5, (c, ma, rl)


def test_row_block_of_three_tails_equals_each_tail_alone():
    """Three slots' tails in one row block: front end + append + chunk attention per slot on
    row pointers and slot-local positions; every slot's cache rows and outputs must be what the
    same tail produces alone."""
    from hipml_b200 import api
    stride, n_rot, theta, eps = 384, 64, 1e7, 1e-6
    tails = [(10, 5), (300, 17), (77, 40)]          # (start position, rows) per slot
    rng = O.Rng(0x7A11)
    slots = len(tails)
    caches = [_filled_cache(rng, stride, start) for start, _ in tails]
    total = sum(n for _, n in tails)
    qg = rng.normals(total * H * 2 * D).reshape(total, H * 2 * D)
    k = rng.normals(total * KV * D).reshape(total, KV * D)
    v = rng.normals(total * KV * D).reshape(total, KV * D)
    qn = (1.0 + rng.normals(D, 0.1)).astype(np.float32)
    kn = (1.0 + rng.normals(D, 0.1)).astype(np.float32)
    dqn, dkn = _dev(qn), _dev(kn)

    def run(rows_qg, rows_k, rows_v, kc, vc, start, n):
        """One tail: returns (attention output, k cache, v cache)."""
        q = torch.empty(n, H * D, device="cuda")
        gate = torch.empty(n, H * D, device="cuda")
        api.attn_front_append_q8(rows_qg, rows_k, rows_v, q, gate, dqn, dkn, kc, vc, H, KV, D, n_rot,
                                 theta, eps, pos0=start, tokens=n, stride=stride)
        ws = torch.empty(api.attn_chunk_workspace_bytes(KV, D, start, n), dtype=torch.uint8,
                         device="cuda")
        out = torch.full((n, H * D), float("nan"), device="cuda")
        api.attn_chunk(q, kc, vc, out, H, KV, D, start, n, 1, stride, None, None, 1, 0, ws)
        return out, q

    # batched: one row block, one cache allocation with a region per slot
    dqg, dk, dv = _dev(qg), _dev(k), _dev(v)
    slot_bytes = KV * stride * ROW
    big_k = torch.empty(slots * slot_bytes, dtype=torch.uint8, device="cuda")
    big_v = torch.empty(slots * slot_bytes, dtype=torch.uint8, device="cuda")
    for s, (kb, vb) in enumerate(caches):
        big_k[s * slot_bytes:(s + 1) * slot_bytes] = _dev(kb).flatten()
        big_v[s * slot_bytes:(s + 1) * slot_bytes] = _dev(vb).flatten()
    batched, first = [], 0
    for s, (start, n) in enumerate(tails):
        kc = big_k[s * slot_bytes:(s + 1) * slot_bytes]
        vc = big_v[s * slot_bytes:(s + 1) * slot_bytes]
        out, q = run(dqg[first:first + n], dk[first:first + n], dv[first:first + n], kc, vc, start, n)
        batched.append((out.cpu().numpy(), kc.cpu().numpy().copy(), vc.cpu().numpy().copy(),
                        q.cpu().numpy()))
        first += n
    assert api.check_device_status() == 0

    # alone: every tail with private copies of its rows and its cache
    first = 0
    for s, (start, n) in enumerate(tails):
        kc, vc = _dev(caches[s][0]).flatten(), _dev(caches[s][1]).flatten()
        out, q = run(_dev(qg[first:first + n]), _dev(k[first:first + n]), _dev(v[first:first + n]), kc,
                     vc, start, n)
        assert np.array_equal(out.cpu().numpy(), batched[s][0]), f"slot {s}: outputs differ"
        assert np.array_equal(kc.cpu().numpy(), batched[s][1]) and np.array_equal(vc.cpu().numpy(),
                                                                                  batched[s][2])
        # and against the oracle: attention of the rotated q rows over the dequantised cache
        rows = start + n
        kq = cases.unpack_head_major(O.dequantize_q8(batched[s][1].reshape(KV, stride, ROW)[:, :rows]),
                                     KV, rows, D)
        vq = cases.unpack_head_major(O.dequantize_q8(batched[s][2].reshape(KV, stride, ROW)[:, :rows]),
                                     KV, rows, D)
        c = cases.ChunkCase(batched[s][3], kq, vq, None, None, H, KV, D, start, n, stride)
        want = cases.chunk_expected(c, threads=4)
        ok, ma, rl = cases.attention_within_bar(want, batched[s][0])
        assert ok, (s, ma, rl)
        # rows past the tail were not touched
        assert np.all(batched[s][1].reshape(KV, stride, ROW)[:, rows:] == 0xA5)
        first += n


def test_prefix_snapshot_and_restore_move_only_the_live_rows():
    from hipml_b200 import api
    stride, live = 400, 150
    rng = O.Rng(0x5A47)
    kb, vb = _filled_cache(rng, stride, live)
    q = rng.normals(H * D)
    dk, dv = _dev(kb), _dev(vb)
    splits = api.decode_splits(live)

    def decode(kc, vc):
        out = torch.full((H * D,), float("nan"), device="cuda")
        acc = torch.empty(H * splits * D, device="cuda")
        ml = torch.empty(H * splits * 2, device="cuda")
        api.attn_decode_kv(_ints([live - 1, live, 0, 0, 0, 0, 0, 0]), _dev(q), kc, vc, acc, ml, out, H,
                           KV, D, stride, SCALE, splits)
        return out.cpu().numpy()

    before = decode(dk, dv)
    snap_k = torch.full((KV * live * ROW,), 0x11, dtype=torch.uint8, device="cuda")
    snap_v = torch.full((KV * live * ROW,), 0x11, dtype=torch.uint8, device="cuda")
    api.kv_rows_copy(snap_k, dk, KV, ROW, live, stride, live)
    api.kv_rows_copy(snap_v, dv, KV, ROW, live, stride, live)
    assert np.array_equal(snap_k.cpu().numpy().reshape(KV, live, ROW), kb[:, :live])
    # another request overwrites the cache, then the prefix comes back
    dk.fill_(0x33)
    dv.fill_(0x33)
    api.kv_rows_copy(dk, snap_k, KV, ROW, stride, live, live)
    api.kv_rows_copy(dv, snap_v, KV, ROW, stride, live, live)
    got_k = dk.cpu().numpy().reshape(KV, stride, ROW)
    assert np.array_equal(got_k[:, :live], kb[:, :live]) and np.all(got_k[:, live:] == 0x33)
    assert np.array_equal(decode(dk, dv), before)
    with pytest.raises(Exception, match="rows copy"):
        api.kv_rows_copy(dk, snap_k, KV, ROW, stride, live, live + 1)
