"""The allocation-free decode entry against the ordinary one.

hipml_attn_decode_kv_static serves callers that cannot allocate device memory (a host
running from a fixed arena, a binding with no device allocator): its split partials live in
an array inside the library instead of caller buffers. It must give what
hipml_attn_decode_kv gives with caller scratch, on consecutive calls that reuse the array
(the second call finds the first call's partials in it), and it must refuse a request that
does not fit the array. Collected last on purpose: the file name sorts after every other test.
"""
import numpy as np
import pytest
import torch

import oracle as O

pytestmark = pytest.mark.gpu


def _step(seq):
    return torch.tensor([seq - 1, seq, 0, 0, 0, 0, 0, 0], dtype=torch.int32, device="cuda")


def _case(seed, heads, n_kv, hd, seq, stride):
    rng = O.Rng(seed)
    q = rng.normals(heads * hd)
    row = hd // 32 * 34
    kb = np.zeros((n_kv, stride, row), dtype=np.uint8)
    vb = np.zeros((n_kv, stride, row), dtype=np.uint8)
    kb[:, :seq] = O.quantize_q8(rng.normals(n_kv * seq * hd)).reshape(n_kv, seq, row)
    vb[:, :seq] = O.quantize_q8(rng.normals(n_kv * seq * hd)).reshape(n_kv, seq, row)
    return (torch.from_numpy(q).cuda(), torch.from_numpy(kb).cuda(), torch.from_numpy(vb).cuda(),
            q, kb, vb)


def test_static_scratch_decode_matches_caller_scratch_decode_twice_in_a_row():
    from hipml_b200 import api
    heads, n_kv, hd, scale = 24, 4, 256, 0.0625
    # two different calls back to back: the second reuses the array the first one filled,
    # with fewer splits, so stale partials of the first call sit beside the live ones
    for seed, seq, stride in ((0xA110C, 3000, 3100), (0xA110D, 777, 800)):
        dq, dk, dv, q, kb, vb = _case(seed, heads, n_kv, hd, seq, stride)
        splits = api.decode_splits(seq)
        ref = torch.zeros(heads * hd, device="cuda")
        acc = torch.zeros(heads * splits * hd, device="cuda")
        ml = torch.zeros(heads * splits * 2, device="cuda")
        api.attn_decode_kv(_step(seq), dq, dk, dv, acc, ml, ref, heads, n_kv, hd, stride, scale,
                           splits)
        got = torch.full((heads * hd,), float("nan"), device="cuda")
        api.attn_decode_kv_static(_step(seq), dq, dk, dv, got, heads, n_kv, hd, stride, scale,
                                  splits)
        torch.cuda.synchronize()
        # same kernels, same inputs, same split count: the two entries agree exactly
        assert torch.equal(got, ref)
        want = O.attn_decode_kv_q8(q, kb, vb, heads, n_kv, hd, seq, scale, stride=stride)
        assert O.max_abs(want, got.cpu().numpy()) <= 2e-5


@pytest.mark.parametrize("selector,hd", [(0, 256), (6, 256), (0, 128)],
                         ids=["tensor_core", "scalar", "head_dim_128"])
def test_static_scratch_decode_takes_no_device_memory(selector, hd):
    """What the entry is for: once it has run on the device (the first call resolves the
    array's address), a call changes neither the driver's free-memory figure nor the
    framework allocator's. The scalar split pass (selector 6, or any head_dim but 256) writes
    and folds all `splits` partial slots, over whatever the previous call left in the array."""
    from hipml_b200 import api
    heads, n_kv, scale, seq, stride = 24, 4, 0.0625, 900, 1000
    dq, dk, dv, q, kb, vb = _case(0xA110E + hd + selector, heads, n_kv, hd, seq, stride)
    splits = api.decode_splits(seq)
    got = torch.full((heads * hd,), float("nan"), device="cuda")
    step = _step(seq)
    api.attn_decode_kv_static(step, dq, dk, dv, got, heads, n_kv, hd, stride, scale, splits,
                              selector=selector)        # warm: address lookup, kernel set-up
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    held0, reserved0 = torch.cuda.memory_allocated(), torch.cuda.memory_reserved()
    for _ in range(3):
        api.attn_decode_kv_static(step, dq, dk, dv, got, heads, n_kv, hd, stride, scale, splits,
                                  selector=selector)
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info()
    assert free1 == free0
    assert torch.cuda.memory_allocated() == held0 and torch.cuda.memory_reserved() == reserved0
    want = O.attn_decode_kv_q8(q, kb, vb, heads, n_kv, hd, seq, scale, stride=stride)
    assert O.max_abs(want, got.cpu().numpy()) <= 2e-5


def test_static_scratch_decode_rejects_what_does_not_fit():
    from hipml_b200 import api, _lib
    z = torch.zeros(64 * 256, device="cuda")
    c = torch.zeros(8 * 16 * 272, dtype=torch.uint8, device="cuda")
    with pytest.raises(_lib.HipmlError, match="exceeds the built-in") as err:
        api.attn_decode_kv_static(_step(1), z, c, c, z, 64, 8, 256, 16, 0.0625, 256)
    assert err.value.code == _lib.ERR_WORKSPACE
