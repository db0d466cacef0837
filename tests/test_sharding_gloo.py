"""The multi-GPU partition on CPU: two gloo ranks stand in for two GPUs.

Each rank holds its range of cache rows, folds them to one (acc, max, sum) triple per head
with a numpy stand-in for the shard kernel, the triples are all-gathered over gloo and folded
with the numpy mirror of the combine kernel; the result must equal the oracle's attention
over the whole cache. The GPU tests check the kernels against the same mirrors.
"""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle as O
from hipml_b200 import sharding

HEADS, N_KV, HD, SEQ, SCALE = 12, 2, 64, 301, 0.125
ROW = HD // 32 * 34


def _inputs():
    rng = O.Rng(0x5EA)
    q = rng.normals(HEADS * HD)
    kb = O.quantize_q8(rng.normals(N_KV * SEQ * HD, 0.3)).reshape(N_KV, SEQ, ROW)
    vb = O.quantize_q8(rng.normals(N_KV * SEQ * HD)).reshape(N_KV, SEQ, ROW)
    return q, kb, vb


def shard_triple(q, kb, vb, lo, n):
    """numpy stand-in for hipml_attn_decode_kv_shard over local rows [lo, lo+n)."""
    out = np.zeros((HEADS, HD + 2), dtype=np.float32)
    out[:, HD] = -np.inf
    if n == 0:
        return out
    group = HEADS // N_KV
    log2e = np.float32(1.4426950408889634)
    for h in range(HEADS):
        k = O.dequantize_q8(kb[h // group, lo:lo + n]).reshape(n, HD)
        v = O.dequantize_q8(vb[h // group, lo:lo + n]).reshape(n, HD)
        s = (k @ q[h * HD:(h + 1) * HD]) * np.float32(SCALE) * log2e
        m = s.max()
        p = np.exp2(s - m).astype(np.float32)
        out[h, :HD] = p @ v
        out[h, HD], out[h, HD + 1] = m, p.sum()
    return out


def _worker(rank, world, port, capacity, seq, result):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    q, kb, vb = _inputs()
    lo, hi = sharding.decode_shard_range(capacity, world, rank)
    n = sharding.local_length(seq, lo, hi)
    mine = torch.from_numpy(shard_triple(q, kb, vb, lo, n))
    gathered = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(gathered, mine)
    out = sharding.fold_triples(torch.stack(gathered).numpy())
    if rank == 0:
        result.put(out)
    dist.barrier()
    dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("capacity,seq", [(SEQ, SEQ), (SEQ, 140), (400, SEQ)])
def test_two_rank_sequence_split_decode_matches_the_oracle(capacity, seq):
    ctx = mp.get_context("spawn")
    result = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, capacity, seq, result)) for r in range(2)]
    for p in procs:
        p.start()
    out = result.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    q, kb, vb = _inputs()
    want = O.attn_decode_kv_q8(q, kb, vb, HEADS, N_KV, HD, seq, SCALE, stride=SEQ)
    assert O.max_abs(want, out.ravel()) < 2e-6


def _prefill_inputs(tokens):
    rng = O.Rng(0x9F1)
    q = rng.normals(tokens * HEADS * HD).reshape(tokens, HEADS * HD)
    k = rng.normals(tokens * N_KV * HD, 0.3).reshape(tokens, N_KV * HD)
    v = rng.normals(tokens * N_KV * HD).reshape(tokens, N_KV * HD)
    return q, k, v


def chunk_rows_numpy(q, k, v, pos0, off, rows):
    """numpy stand-in for the chunk attention of query rows [pos0 + off, pos0 + off + rows):
    row t sees cache rows 0 .. t inclusive (the position is on the query side only)."""
    group = HEADS // N_KV
    out = np.zeros((rows, HEADS * HD), dtype=np.float32)
    for r in range(rows):
        t = pos0 + off + r
        for h in range(HEADS):
            kv = h // group
            kk = k[:t + 1, kv * HD:(kv + 1) * HD].astype(np.float64)
            vv = v[:t + 1, kv * HD:(kv + 1) * HD].astype(np.float64)
            s = kk @ q[t, h * HD:(h + 1) * HD].astype(np.float64) * SCALE
            w = np.exp(s - s.max())
            out[r, h * HD:(h + 1) * HD] = (w / w.sum()) @ vv
    return out


def _prefill_worker(rank, world, port, tokens, chunk, by_chunks, result):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    q, k, v = _prefill_inputs(tokens)
    chunks = [(p, min(chunk, tokens - p)) for p in range(0, tokens, chunk)]
    mine = np.full((tokens, HEADS * HD), np.nan, dtype=np.float32)
    work = 0
    for ci, (p, n) in enumerate(chunks):
        off, rows = (sharding.chunk_part(ci, len(chunks), n, world, rank) if by_chunks
                     else sharding.query_part(ci, n, world, rank))
        if rows > 0:
            mine[p + off:p + off + rows] = chunk_rows_numpy(q, k, v, p, off, rows)
            work += rows * (p + off) + rows * (rows + 1) // 2
    parts = [torch.empty(tokens, HEADS * HD) for _ in range(world)]
    dist.all_gather(parts, torch.from_numpy(mine))
    works = [torch.zeros(1, dtype=torch.int64) for _ in range(world)]
    dist.all_gather(works, torch.tensor([work]))
    if rank == 0:
        result.put((torch.stack(parts).numpy(), [int(w.item()) for w in works]))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("tokens,chunk,by_chunks", [(64, 16, True), (75, 16, True), (75, 16, False)],
                         ids=["4_chunks_in_pairs", "5_chunks_middle_split", "row_halves"])
def test_two_ranks_that_share_the_kv_heads_cover_the_prefill_once(tokens, chunk, by_chunks):
    """The 8-GPU prefill partition on two gloo ranks: the ranks that share a KV head divide the
    chunks in pairs (or every chunk's rows); no exchange. Every output row is produced by
    exactly one rank, the merged rows equal the oracle's causal attention over the whole job,
    and the ranks' causal work is balanced."""
    ctx = mp.get_context("spawn")
    result = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_prefill_worker, args=(r, 2, port, tokens, chunk, by_chunks, result))
             for r in range(2)]
    for p in procs:
        p.start()
    parts, works = result.get(timeout=180)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    owned = ~np.isnan(parts[:, :, 0])
    assert np.all(owned.sum(axis=0) == 1), "a row was produced twice or not at all"
    merged = np.where(np.isnan(parts[0]), parts[1], parts[0])
    q, k, v = _prefill_inputs(tokens)
    want = O.attn_chunk_f32(q, k, v, HEADS, N_KV, HD, 0, tokens, SCALE)
    assert O.max_abs(want.ravel(), merged.ravel()) < 2e-5
    if tokens % chunk == 0:       # (a ragged last chunk makes its pair lighter at this tiny size)
        assert max(works) <= 1.06 * sum(works) / 2, works


def test_partition_arithmetic():
    # decode ranges tile [0, capacity) in order; each position has exactly one owner
    for cap, world in [(100000, 8), (100136, 4), (7, 8), (672, 2)]:
        edges = [sharding.decode_shard_range(cap, world, r) for r in range(world)]
        assert edges[0][0] == 0 and edges[-1][1] == cap
        assert all(a[1] == b[0] for a, b in zip(edges, edges[1:]))
        assert max(hi - lo for lo, hi in edges) - min(hi - lo for lo, hi in edges) <= 1
        for pos in (0, cap // 2, cap - 1):
            r = sharding.decode_owner(pos, cap, world)
            assert edges[r][0] <= pos < edges[r][1]
        assert sum(sharding.local_length(cap - 3, lo, hi) for lo, hi in edges) == cap - 3
    # prefill: KV heads first, then query halves that rotate with the chunk index
    assert sharding.kv_head_shard(24, 4, 1, 0) == (1, 1, 0, 0, 4, 24)
    assert sharding.kv_head_shard(24, 4, 4, 3) == (4, 1, 3, 0, 1, 6)
    assert sharding.kv_head_shard(24, 4, 8, 6) == (4, 2, 2, 1, 1, 6)
    with pytest.raises(ValueError):
        sharding.kv_head_shard(24, 4, 3, 0)
    for ci in range(4):
        parts = [sharding.query_part(ci, 2048, 2, qi) for qi in range(2)]
        assert sorted(parts) == [(0, 1024), (1024, 1024)]
    assert sharding.query_part(0, 2048, 2, 0) != sharding.query_part(1, 2048, 2, 0)
    parts = sorted(sharding.query_part(0, 1697, 2, qi) for qi in range(2))
    assert parts == [(0, 849), (849, 848)]
    # or whole chunks, dealt out in pairs (i, n-1-i) of equal causal cost; what does not divide
    # (a pair beyond a multiple of the rank count, the middle chunk) is split by rows
    for n_chunks, tokens in ((4, 8192), (49, 100000), (5, 10240), (2, 4096), (1, 100)):
        chunks = [(p, min(2048, tokens - p)) for p in range(0, tokens, 2048)]
        assert len(chunks) == n_chunks
        work = [0, 0]
        whole = 0
        for ci, (p, n) in enumerate(chunks):
            owned = [sharding.chunk_part(ci, n_chunks, n, 2, qi) for qi in range(2)]
            covered = sorted((off, off + rows) for off, rows in owned if rows)
            assert covered[0][0] == 0 and covered[-1][1] == n           # every row once
            assert all(a[1] == b[0] for a, b in zip(covered, covered[1:]))
            whole += len(covered) == 1
            for qi, (off, rows) in enumerate(owned):                    # causal (query, key) pairs
                work[qi] += rows * (p + off) + rows * (rows + 1) // 2
        assert whole == n_chunks // 4 * 4
        assert max(work) <= 1.02 * sum(work) / 2 or n_chunks < 4
    assert [sharding.chunk_part(ci, 4, 2048, 2, 0)[1] for ci in range(4)] == [2048, 0, 0, 2048]
    assert sharding.chunk_part(3, 4, 2048, 1, 0) == (0, 2048)


def test_fold_handles_empty_shards():
    g = np.zeros((3, 2, 6), dtype=np.float32)
    g[:, :, 4] = -np.inf
    assert np.all(sharding.fold_triples(g) == 0.0)
    g[1, :, :4] = [2.0, 4.0, 6.0, 8.0]
    g[1, :, 4], g[1, :, 5] = 0.5, 2.0
    assert np.allclose(sharding.fold_triples(g), [[1.0, 2.0, 3.0, 4.0]] * 2)


def test_prefill_key_split_policy_fills_two_waves():
    """A rank with all 4 KV heads runs unsplit; fewer local pairs get more key slices."""
    from hipml_b200 import sharding
    assert sharding.prefill_key_splits(2048, 6, 4) == 1
    assert sharding.prefill_key_splits(2048, 6, 2) == 2
    assert sharding.prefill_key_splits(2048, 6, 1) == 3
    assert sharding.prefill_key_splits(1024, 6, 1) == 6
    assert sharding.prefill_key_splits(1, 6, 1) == 8          # capped
    assert sharding.prefill_key_splits(100000, 6, 4) == 1
    # with the position the count comes from the launch cost model: the measured optima
    assert [sharding.prefill_key_splits(2048, 6, 1, pos0=p) for p in (0, 2048, 4096, 6144)] == [2, 3, 3, 3]
    assert [sharding.prefill_key_splits(2048, 6, 2, pos0=p) for p in (0, 2048, 6144)] == [1, 1, 3]
    assert [sharding.prefill_key_splits(2048, 6, 4, pos0=p) for p in (0, 2048, 4096, 6144)] == [1, 1, 1, 1]
    assert sharding.prefill_key_splits(64, 6, 1, pos0=0) == 1
    # the estimate itself: unsliced, four KV heads, first chunk (measured 154 us)
    assert 130 < sharding.chunk_launch_estimate_us(2048, 6, 4, 0, 1) < 170
