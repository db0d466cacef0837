"""The multi-slot decode plan on the host: hipml_decode_plan_quota runs the same solver the
kernels run on the device (one template, two instantiations). Whatever the live lengths are,
the plan's runs must fit the CTAs that are launched: a CTA takes exactly one run, so a run
past the grid would never be computed."""
import random

from hipml_b200 import api


def _runs(lens, quota, n_kv):
    return sum(max(1, -(-(-(-n // 64)) // quota)) for n in lens) * n_kv


def _batch_splits(stride, slots):
    return api.batch_splits(stride, slots)


def test_quota_fits_the_grid_for_every_length_up_to_the_context_limit():
    rng = random.Random(7)
    cta_slots, n_kv = 296, 4
    cases = [[150_000] * 16, [200_000] * 16, [100_000] * 32, [262_144] * 37, [1] * 37, [0] * 5,
             [262_144] + [1] * 36, [64] * 20 + [65] * 17]
    for _ in range(300):
        slots = rng.randint(2, 37)   # the plan is taken while 2 * slots * n_kv <= cta_slots
        top = rng.choice([100, 5_000, 70_000, 262_144])
        cases.append([rng.randint(0, top) for _ in range(slots)])
    for lens in cases:
        slots = len(lens)
        assert 2 * slots * n_kv <= cta_slots
        splits = _batch_splits(max(max(lens), 1) + 8, slots)
        quota = api.decode_plan_quota(lens, splits, n_kv, cta_slots)
        assert quota >= 1
        assert _runs(lens, quota, n_kv) <= cta_slots, (lens, quota)
        # no slot needs more partial slots than its scratch has
        assert all(max(1, -(-(-(-n // 64)) // quota)) <= splits for n in lens)
        # and the quota is the smallest that does both
        if quota > 1:
            longest = max(-(-n // 64) for n in lens)
            floor_q = max(-(-longest // splits), 1)
            assert quota == floor_q or _runs(lens, quota - 1, n_kv) > cta_slots, (lens, quota)


def test_quota_matches_the_earlier_upward_scan_where_that_converged():
    """Before the solver was a bisection it scanned upwards from the first guess; where that
    scan ended within its step limit both give the same plan (same partition, same bits)."""
    rng = random.Random(11)
    cta_slots, n_kv = 296, 4
    for _ in range(200):
        slots = rng.randint(2, 16)
        lens = [rng.randint(1, 8192) for _ in range(slots)]
        splits = _batch_splits(8448, slots)
        tiles = [-(-n // 64) for n in lens]
        q = max(-(-sum(tiles) * n_kv // cta_slots), -(-max(tiles) // splits), 1)
        for _step in range(64):
            if q >= max(tiles) or sum(-(-t // q) for t in tiles) * n_kv <= cta_slots:
                break
            q += 1
        assert api.decode_plan_quota(lens, splits, n_kv, cta_slots) == q


def test_quota_rejects_arguments_outside_the_plan():
    assert api.decode_plan_quota([100, 200], 4, 4, 8) == -1   # 2 * slots * n_kv > cta_slots
