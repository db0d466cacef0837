"""Host arithmetic of the multi-GPU partition of the attention path (one process per GPU).

The reference is single-GPU; what it has is split-K over the key axis inside one GPU, with
unnormalised (acc, max, sum) partials and an associative fold
(crates/hipml-kernels/kernels/attn_decode_kv.hip:491-532). The partition here lifts that
split index from thread blocks to ranks:

* prefill shards by KV head (ranks <= n_kv): each rank owns n_kv/ranks KV heads and their
  query heads; no exchange inside the attention. Beyond n_kv ranks, the ranks that share a
  KV head take alternating halves of every chunk's query rows (still no exchange; the K/V
  append of the chunk is repeated on each of them).
* decode shards by sequence: rank r holds cache rows [lo_r, hi_r) of every KV head; the new
  token's row is appended on the rank that owns its position; every rank folds its rows to
  one (acc, max, sum) triple per head; the triples are all-gathered (NCCL) and folded again.

Only integers and numpy here; the GPU work is in libhipml_cuda.so.
"""
from __future__ import annotations

import numpy as np


def kv_head_shard(n_heads: int, n_kv: int, world: int, rank: int):
    """(kv_shards, q_shards, kv_index, q_index, local_n_kv, local_n_heads) of `rank`."""
    kv_shards = min(world, n_kv)
    if n_kv % kv_shards or world % kv_shards:
        raise ValueError(f"world {world} does not tile n_kv {n_kv}")
    q_shards = world // kv_shards
    return (kv_shards, q_shards, rank % kv_shards, rank // kv_shards, n_kv // kv_shards,
            n_heads // kv_shards)


def query_part(chunk_index: int, chunk_rows: int, q_shards: int, q_index: int):
    """(row offset, rows) of this rank's share of a chunk's query rows: contiguous parts that
    rotate with the chunk index so every rank sees the same causal work."""
    base, extra = divmod(chunk_rows, q_shards)
    part = (q_index + chunk_index) % q_shards
    start = part * base + min(part, extra)
    return start, base + (1 if part < extra else 0)


def chunk_part(chunk_index: int, n_chunks: int, chunk_rows: int, q_shards: int, q_index: int):
    """(row offset, rows) of this rank's share of chunk `chunk_index` when the ranks that share
    a KV head divide the CHUNKS of a prefill among themselves instead of every chunk's rows:
    (0, chunk_rows) for a chunk the rank owns, (0, 0) for one it leaves to another rank. A chunk
    at position p costs about p + chunk/2 key rows per query row, so chunks are dealt out in
    pairs (i, n-1-i) of equal cost, the pairs going round the ranks: every rank gets the same
    causal work, and every chunk it attends is a whole chunk (twice the query tiles of half a
    chunk, so half the key slices and combine passes). What does not divide - the pairs beyond
    a multiple of q_shards and the middle chunk of an odd count - is split by rows as
    query_part does. The rank still appends every chunk's K/V rows to its cache: a later chunk
    of its own reads them."""
    if q_shards <= 1:
        return 0, chunk_rows
    pair = min(chunk_index, n_chunks - 1 - chunk_index)
    whole_pairs = (n_chunks // 2) // q_shards * q_shards
    if pair >= whole_pairs:
        return query_part(chunk_index, chunk_rows, q_shards, q_index)
    return (0, chunk_rows) if pair % q_shards == q_index else (0, 0)


def decode_shard_range(capacity: int, world: int, rank: int):
    """Cache rows [lo, hi) of every KV head that `rank` holds, for a context of `capacity`
    rows: contiguous, as even as possible."""
    base, extra = divmod(capacity, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def decode_owner(pos: int, capacity: int, world: int) -> int:
    """The rank whose range holds global position `pos`."""
    for r in range(world):
        lo, hi = decode_shard_range(capacity, world, r)
        if lo <= pos < hi:
            return r
    raise ValueError(f"position {pos} beyond capacity {capacity}")


def local_length(seq: int, lo: int, hi: int) -> int:
    """How many of the first `seq` global positions fall in [lo, hi)."""
    return max(0, min(seq, hi) - lo)


def fold_triples(gathered: np.ndarray) -> np.ndarray:
    """numpy mirror of hipml_attn_decode_combine: gathered [shards][heads][D+2] =
    (acc, max_log2, sum) -> out [heads][D]. Used by the CPU tests of the exchange."""
    g = np.asarray(gathered, dtype=np.float32)
    acc, m, l = g[..., :-2], g[..., -2], g[..., -1]
    big = m.max(axis=0)
    with np.errstate(invalid="ignore"):
        w = np.where(np.isneginf(m), np.float32(0), np.exp2(m - big[None, :])).astype(np.float32)
    num = (acc * w[..., None]).sum(axis=0)
    den = (l * w).sum(axis=0)
    with np.errstate(invalid="ignore", divide="ignore"):
        out = np.where(den[:, None] > 0, num / den[:, None], np.float32(0))
    return out.astype(np.float32)


# Cost model of one launch of the tensor-core chunk kernel (B200, measured with a per-CTA time
# line): a CTA pair spends ~13 us outside its key-tile loop and 4.4 us per 128-key tile in it;
# slicing the key axis adds a combine pass, the partials' round trip and a launch (~30 us).
PAIR_FIXED_US, PAIR_STEP_US, SLICED_EXTRA_US = 13.0, 4.4, 30.0


def chunk_launch_estimate_us(chunk_rows: int, group: int, local_n_kv: int, pos0: int, slices: int,
                             sm_pairs: int = 74) -> float:
    """Estimated duration of the chunk attention of `chunk_rows` query rows at position `pos0`
    with `slices` key slices per query tile, for a rank that owns `local_n_kv` KV heads: the
    jobs (one per pair of query tiles, KV head and slice) are dealt to the device's SM pairs
    longest first, as the launch order does."""
    qtile = max(128 // group, 1)
    tiles = -(-chunk_rows // qtile)
    jobs = []
    for pair in range(-(-tiles // 2)):
        last_query = min((2 * pair + 2) * qtile, chunk_rows)
        key_tiles = -(-(pos0 + last_query) // 128)
        for sl in range(slices):
            lo, hi = key_tiles * sl // slices, key_tiles * (sl + 1) // slices
            jobs.append(PAIR_FIXED_US + PAIR_STEP_US * (hi - lo))
    jobs = sorted(jobs * local_n_kv, reverse=True)
    slots = [0.0] * sm_pairs
    for job in jobs:
        k = min(range(sm_pairs), key=slots.__getitem__)
        slots[k] += job
    return max(slots) + (SLICED_EXTRA_US if slices > 1 else 0.0)


def prefill_key_splits(chunk_rows: int, group: int, local_n_kv: int, sm_pairs: int = 74,
                       pos0: int | None = None) -> int:
    """Key slices per query tile for a rank's share of a prefill chunk. The tensor-core chunk
    kernel runs one CTA pair per two query tiles of 128 // group queries; a rank that owns
    all 4 KV heads has more pairs than SM pairs and runs unsplit, a rank with fewer pairs cuts
    the key axis so that about two waves of the device are filled (measured on the 2048-token
    chunk: 1 / 2 / 3 slices are the fastest for 4 / 2 / 1 local KV heads). With the chunk's
    position given the count comes from the cost model above instead: the first chunk of a
    prefill, whose query tiles see 1 - 16 key tiles, wants fewer slices than the later ones
    (measured, 2048 rows: one KV head 2 / 3 / 3 / 3 slices at positions 0 / 2048 / 4096 / 6144,
    two KV heads 1 / 1 / 2 - 3 / 3, four KV heads 1 up to 8,192 keys; the model picks the same)."""
    qtile = max(128 // group, 1)
    pairs = -(-(-(-chunk_rows // qtile)) // 2) * local_n_kv
    if pos0 is None:
        if pairs >= 2 * sm_pairs:
            return 1
        return max(1, min(8, round(2 * sm_pairs / pairs)))
    # (deep chunks: the jobs are long and alike, so what matters is that jobs / SM pairs comes
    # out just under a whole number - 196, 98 or 49 pairs x 3 slices = 7.9, 4.0, 2.0 rounds;
    # measured on the 100,000-token prefill: 302 -> 289 ms per layer with all four KV heads,
    # 150 -> 142 ms with two, 3 the best of 2 .. 8 with one)
    best, best_us = 1, None
    for slices in range(1, 7):
        us = chunk_launch_estimate_us(chunk_rows, group, local_n_kv, pos0, slices, sm_pairs)
        if best_us is None or us < best_us - 1e-9:
            best, best_us = slices, us
    return best
