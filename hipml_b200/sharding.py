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


def prefill_key_splits(chunk_rows: int, group: int, local_n_kv: int, sm_pairs: int = 74,
                       pos0: int | None = None) -> int:
    """Key slices per query tile for a rank's share of a prefill chunk. The tensor-core chunk
    kernel runs one CTA pair per two query tiles of 128 // group queries; a rank that owns
    all 4 KV heads has more pairs than SM pairs and runs unsplit, a rank with fewer pairs cuts
    the key axis so that about two waves of the device are filled (measured on the 2048-token
    chunk: 1 / 2 / 3 slices are the fastest for 4 / 2 / 1 local KV heads). With the chunk's
    position given, a slice also keeps at least about four 128-key tiles on average: a CTA
    pair costs ~13 us besides its 4.4 us per key tile, and the first chunk of a prefill, whose
    query tiles see 8.5 key tiles on average, is faster in 2 slices than in 3 (66 against 81 us
    for one KV head, measured)."""
    qtile = max(128 // group, 1)
    pairs = -(-(-(-chunk_rows // qtile)) // 2) * local_n_kv
    if pairs >= 2 * sm_pairs:
        return 1
    fill = max(1, min(8, round(2 * sm_pairs / pairs)))
    if pos0 is None:
        return fill
    mean_tiles = (pos0 + chunk_rows / 2) / 128
    return max(1, min(fill, int(mean_tiles // 4)))
