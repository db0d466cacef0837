"""The reference's seeded parity cases for the attention path, restated.

Each builder draws its inputs from the reference's generator in the reference's draw
order, so the inputs are the ones `hipml parity` / `hipml attn-parity` would use:
  * q8 decode cases and the 100K deep case: crates/hipml-core/src/parity_kv.rs:68-246
    (draw order q, then K with normal_scaled(0.3), then V; the cache is quantised on the
    host and both sides read the same bytes);
  * kv_encode_q8: crates/hipml-core/src/parity.rs:364-378,660-681;
  * chunk attention 37 queries at position 29: crates/hipml-cli/src/attn_chunk_parity.rs:
    24-58 (f32 cache) and :124-207 (q8 cache, optional pad so stride > live length);
  * f32 position-major decode: crates/hipml-core/src/attn_parity.rs:101-161.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

import oracle as O


@dataclass(frozen=True)
class KvCase:
    name: str
    heads: int
    n_kv: int
    dim: int
    seq: int
    splits: int
    scale: float
    seed: int
    dtype: int = 0      # KvDtype::id(): 0 = q8_0, 1 = q4_0


# parity_kv.rs:68-215, the q8 rows
KV_CASES = [
    KvCase("attn_decode_kv_q8_hd256_s1", 6, 1, 256, 1, 1, 0.0625, 0x9E00_0001),
    KvCase("attn_decode_kv_q8_hd256_s37", 6, 1, 256, 37, 1, 0.0625, 0x9E00_0002),
    KvCase("attn_decode_kv_q8_hd256_s1000", 6, 1, 256, 1000, 7, 0.0625, 0x9E00_0003),
    KvCase("attn_decode_kv_q8_hd256_s4096", 6, 1, 256, 4096, 16, 0.0625, 0x9E00_0004),
    KvCase("attn_decode_kv_q8_hd64_s37", 8, 2, 64, 37, 1, 0.125, 0x9E00_0009),
    KvCase("attn_decode_kv_q8_hd64_s1000", 8, 2, 64, 1000, 7, 0.125, 0x9E00_000A),
]

# parity_kv.rs:68-215, the q4 rows
KV_CASES_Q4 = [
    KvCase("attn_decode_kv_q4_hd256_s1", 6, 1, 256, 1, 1, 0.0625, 0x9E00_0005, 1),
    KvCase("attn_decode_kv_q4_hd256_s37", 6, 1, 256, 37, 1, 0.0625, 0x9E00_0006, 1),
    KvCase("attn_decode_kv_q4_hd256_s1000", 6, 1, 256, 1000, 7, 0.0625, 0x9E00_0007, 1),
    KvCase("attn_decode_kv_q4_hd256_s4096", 6, 1, 256, 4096, 16, 0.0625, 0x9E00_0008, 1),
    KvCase("attn_decode_kv_q4_hd64_s37", 8, 2, 64, 37, 1, 0.125, 0x9E00_000B, 1),
    KvCase("attn_decode_kv_q4_hd64_s1000", 8, 2, 64, 1000, 7, 0.125, 0x9E00_000C, 1),
]

# parity_kv.rs:219-246
DEEP_CASE = KvCase("attn_decode_kv_q8_hd256_s100000", 1, 1, 256, 100000, 256, 0.0625, 0x9E00_1001)
DEEP_CASE_Q4 = KvCase("attn_decode_kv_q4_hd256_s100000", 1, 1, 256, 100000, 64, 0.0625, 0x9E00_1002, 1)


def kv_case_inputs(c: KvCase):
    """(q [heads*dim] f32, k bytes, v bytes) with the cache encoded on the host."""
    rng = O.Rng(c.seed)
    q = rng.normals(c.heads * c.dim)
    kf = rng.normals(c.n_kv * c.seq * c.dim, 0.3)
    vf = rng.normals(c.n_kv * c.seq * c.dim)
    quantize = O.quantize_q4 if c.dtype == 1 else O.quantize_q8
    return q, quantize(kf), quantize(vf)


def kv_case_expected(c: KvCase, q, kb, vb):
    return O.attn_decode_kv(q, kb, vb, c.dtype, c.heads, c.n_kv, c.dim, c.seq, c.scale)


# parity.rs:364-378
KV_ENCODE_CASE = dict(n_kv=4, head_dim=64, seq=8, pos=3, seed=0xDDDD_EEEE_FFFF_0003)


def kv_encode_case_inputs():
    c = KV_ENCODE_CASE
    rng = O.Rng(c["seed"])
    width = c["n_kv"] * c["head_dim"]
    k = rng.normals(width, 1.5)
    v = rng.normals(width, 1.5)
    return k, v


def kv_encode_expected_bytes(k, v, n_kv, head_dim):
    """Per-head row bytes the host format definition writes (K rows then V rows)."""
    rows = []
    for src in (k, v):
        rows.append([O.quantize_q8(src[h * head_dim:(h + 1) * head_dim]) for h in range(n_kv)])
    return rows


def pack_head_major(pos_major: np.ndarray, n_kv: int, seq: int, hd: int) -> np.ndarray:
    """[seq][n_kv*hd] -> [n_kv][seq][hd] (attn_chunk_parity.rs:153-161)."""
    return np.ascontiguousarray(pos_major.reshape(seq, n_kv, hd).transpose(1, 0, 2))


def unpack_head_major(head_major: np.ndarray, n_kv: int, seq: int, hd: int) -> np.ndarray:
    return np.ascontiguousarray(head_major.reshape(n_kv, seq, hd).transpose(1, 0, 2)).reshape(
        seq, n_kv * hd)


@dataclass
class ChunkCase:
    q: np.ndarray          # [tok][heads*hd]
    k: np.ndarray          # f32 position-major [seq][n_kv*hd] (dequantised values for q8)
    v: np.ndarray
    kb: np.ndarray | None  # q8 bytes, head-major with `stride` rows per head
    vb: np.ndarray | None
    heads: int
    n_kv: int
    hd: int
    pos0: int
    tok: int
    stride: int


def chunk_case_f32(heads=24, n_kv=4, hd=256, tok=37, pos0=29, seed=0xC4A0_1234_5678) -> ChunkCase:
    """attn_chunk_parity.rs:24-58."""
    seq = pos0 + tok
    width, nhd = n_kv * hd, heads * hd
    rng = O.Rng(seed)
    q = rng.normals(tok * nhd).reshape(tok, nhd)
    k = rng.normals(seq * width).reshape(seq, width)
    v = rng.normals(seq * width).reshape(seq, width)
    return ChunkCase(q, k, v, None, None, heads, n_kv, hd, pos0, tok, seq)


def chunk_case_q8(heads=24, n_kv=4, hd=256, tok=37, pos0=29, pad=0,
                  seed=0xC4A0_9876_5432, q4=False) -> ChunkCase:
    """attn_chunk_parity.rs:124-207: the cache has stride = pos0 + tok + pad rows per head and
    is drawn and quantised over the whole stride; the oracle reads the dequantised values.
    `q4` quantises the same draws as q4_0 instead."""
    quantize, dequantize = (O.quantize_q4, O.dequantize_q4) if q4 else (O.quantize_q8, O.dequantize_q8)
    stride = pos0 + tok + pad
    width, nhd = n_kv * hd, heads * hd
    rng = O.Rng(seed)
    q = rng.normals(tok * nhd).reshape(tok, nhd)
    kc = rng.normals(stride * width).reshape(stride, width)
    vc = rng.normals(stride * width).reshape(stride, width)
    kb = quantize(pack_head_major(kc, n_kv, stride, hd))
    vb = quantize(pack_head_major(vc, n_kv, stride, hd))
    kq = unpack_head_major(dequantize(kb), n_kv, stride, hd)
    vq = unpack_head_major(dequantize(vb), n_kv, stride, hd)
    return ChunkCase(q, kq, vq, kb, vb, heads, n_kv, hd, pos0, tok, stride)


def chunk_expected(c: ChunkCase, rows=None, threads: int = 1) -> np.ndarray:
    """Oracle rows of a chunk case ([tok][heads*hd]); `rows` = (row0, row_step) samples."""
    scale = np.float32(1.0) / np.sqrt(np.float32(c.hd))
    row0, step = rows if rows else (0, 1)
    return O.attn_chunk_f32(c.q, c.k, c.v, c.heads, c.n_kv, c.hd, c.pos0, c.tok, float(scale),
                            row0=row0, row_step=step, threads=threads)


# attn_parity.rs:101-161 (attn_decode_pm_f32 / attn_decode_split_f32)
def decode_f32_case(seed=0x7777_8888_9999_AAAA):
    n_heads, n_kv, hd, seq, scale = 8, 2, 64, 37, 0.125
    rng = O.Rng(seed)
    q = rng.normals(n_heads * hd)
    k = rng.normals(seq * n_kv * hd, 0.3)
    v = rng.normals(seq * n_kv * hd)
    expected = O.attn_causal_f32(q, k, v, n_heads, n_kv, hd, seq, scale)
    return dict(q=q, k=k, v=v, n_heads=n_heads, n_kv=n_kv, hd=hd, seq=seq, scale=scale,
                expected=expected)


# The acceptance bar of this build for attention outputs, against the f32 oracle.
MAX_ABS = 2e-3
REL_L2 = 1e-4


def attention_within_bar(expected, actual) -> tuple[bool, float, float]:
    ma, rl = O.max_abs(expected, actual), O.rel_l2(expected, actual)
    return (ma <= MAX_ABS and rl <= REL_L2), ma, rl
