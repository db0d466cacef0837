"""ctypes view of the CPU oracle (``hipml_oracle.c``): TEST INFRASTRUCTURE ONLY.

The oracle restates the reference's CPU definition of the attention hot path
(crates/hipml-core/src/{kv,rng,attention,ops,parity}.rs). Only the tests, the
smoke check and the bench's CPU-baseline leg import this module; the product
package never does.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "libhipml_oracle.so")

BLOCK = 32
Q8_BLOCK_BYTES = 34
Q4_BLOCK_BYTES = 18


def build(force: bool = False) -> str:
    """Compile the oracle with the committed Makefile; returns the library path."""
    src = os.path.join(_HERE, "hipml_oracle.c")
    stale = (not os.path.exists(_SO)) or os.path.getmtime(_SO) < os.path.getmtime(src)
    if force or stale:
        subprocess.check_call(["make", "-s", "-C", _HERE])
    return _SO


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        _lib = C.CDLL(build())
        f32p, u8p, u64p = C.POINTER(C.c_float), C.POINTER(C.c_uint8), C.POINTER(C.c_uint64)
        L = _lib
        L.hipml_oracle_f16_to_f32.restype = C.c_float
        L.hipml_oracle_f16_to_f32.argtypes = [C.c_uint16]
        L.hipml_oracle_f32_to_f16.restype = C.c_uint16
        L.hipml_oracle_f32_to_f16.argtypes = [C.c_float]
        L.hipml_oracle_quantize_q8.argtypes = [f32p, C.c_size_t, u8p]
        L.hipml_oracle_dequantize_q8.argtypes = [u8p, C.c_size_t, f32p]
        L.hipml_oracle_synthetic_blocks_q8.argtypes = [C.c_size_t, C.c_uint64, u8p]
        L.hipml_oracle_rng_new.restype = C.c_uint64
        L.hipml_oracle_rng_new.argtypes = [C.c_uint64]
        L.hipml_oracle_rng_next_u64.restype = C.c_uint64
        L.hipml_oracle_rng_next_u64.argtypes = [u64p]
        L.hipml_oracle_rng_uniform.restype = C.c_float
        L.hipml_oracle_rng_uniform.argtypes = [u64p]
        L.hipml_oracle_rng_normal.restype = C.c_float
        L.hipml_oracle_rng_normal.argtypes = [u64p]
        L.hipml_oracle_rng_fill_normal.argtypes = [u64p, C.c_float, f32p, C.c_size_t]
        L.hipml_oracle_attn_causal_f32.argtypes = [f32p, f32p, f32p, C.c_int, C.c_int, C.c_int,
                                                   C.c_int, C.c_float, f32p]
        L.hipml_oracle_attn_chunk_f32.argtypes = [f32p, f32p, f32p, C.c_int, C.c_int, C.c_int,
                                                  C.c_int, C.c_int, C.c_float, f32p, C.c_int,
                                                  C.c_int, C.c_int]
        L.hipml_oracle_attn_decode_kv_q8.argtypes = [f32p, u8p, u8p, C.c_int, C.c_int, C.c_int,
                                                     C.c_int, C.c_float, f32p]
        L.hipml_oracle_attn_decode_kv_q8_strided.argtypes = [f32p, u8p, u8p, C.c_int, C.c_int,
                                                             C.c_int, C.c_int, C.c_int, C.c_float,
                                                             f32p]
        L.hipml_oracle_attn_decode_f32.argtypes = [f32p, f32p, f32p, C.c_int, C.c_int, C.c_int,
                                                   C.c_int, C.c_float, f32p]
        L.hipml_oracle_kv_append_f32.argtypes = [f32p, f32p, f32p, f32p, C.c_size_t, C.c_size_t]
        L.hipml_oracle_compare.argtypes = [f32p, f32p, C.c_size_t, f32p, f32p]
        i4 = C.POINTER(C.c_int)
        L.hipml_oracle_quantize_q4.argtypes = [f32p, C.c_size_t, u8p]
        L.hipml_oracle_dequantize_q4.argtypes = [u8p, C.c_size_t, f32p]
        L.hipml_oracle_synthetic_blocks_q4.argtypes = [C.c_size_t, C.c_uint64, u8p]
        L.hipml_oracle_attn_decode_kv_strided.argtypes = [f32p, u8p, u8p, C.c_int, C.c_int, C.c_int,
                                                          C.c_int, C.c_int, C.c_int, C.c_float, f32p]
        L.hipml_oracle_head_rmsnorm_f32.argtypes = [f32p, f32p, C.c_int, C.c_int, C.c_float, f32p]
        L.hipml_oracle_rope_multi_f32.argtypes = [f32p, C.c_int, C.c_int, C.c_int, i4, i4, C.c_float,
                                                  f32p]
        L.hipml_oracle_rope_neox_f32.argtypes = [f32p, C.c_int, C.c_int, C.c_int, C.c_float, f32p]
        L.hipml_oracle_qg_split_f32.argtypes = [f32p, C.c_int, C.c_int, f32p, f32p]
        L.hipml_oracle_q_gate_f32.argtypes = [f32p, f32p, C.c_size_t, f32p]
    return _lib


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _u8(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.uint8)


def _p(a: np.ndarray, ty):
    return a.ctypes.data_as(C.POINTER(ty))


def f16_to_f32(h: int) -> float:
    return float(lib().hipml_oracle_f16_to_f32(h))


def f32_to_f16(v: float) -> int:
    return int(lib().hipml_oracle_f32_to_f16(C.c_float(v)))


def quantize_q8(values) -> np.ndarray:
    """kv::quantize(Q8, values): flat f32 (multiple of 32) -> bytes."""
    v = _f32(values).ravel()
    assert v.size % BLOCK == 0, "values must be a multiple of 32"
    out = np.empty(v.size // BLOCK * Q8_BLOCK_BYTES, dtype=np.uint8)
    lib().hipml_oracle_quantize_q8(_p(v, C.c_float), v.size, _p(out, C.c_uint8))
    return out


def dequantize_q8(data) -> np.ndarray:
    b = _u8(data).ravel()
    assert b.size % Q8_BLOCK_BYTES == 0, "truncated block"
    out = np.empty(b.size // Q8_BLOCK_BYTES * BLOCK, dtype=np.float32)
    lib().hipml_oracle_dequantize_q8(_p(b, C.c_uint8), b.size, _p(out, C.c_float))
    return out


def synthetic_blocks_q8(n_blocks: int, seed: int) -> np.ndarray:
    out = np.empty(n_blocks * Q8_BLOCK_BYTES, dtype=np.uint8)
    lib().hipml_oracle_synthetic_blocks_q8(n_blocks, C.c_uint64(seed), _p(out, C.c_uint8))
    return out


class Rng:
    """The reference's xorshift64* + Box-Muller generator (rng.rs)."""

    def __init__(self, seed: int):
        self._s = C.c_uint64(lib().hipml_oracle_rng_new(C.c_uint64(seed & (2**64 - 1))))

    def next_u64(self) -> int:
        return int(lib().hipml_oracle_rng_next_u64(C.byref(self._s)))

    def uniform(self) -> float:
        return float(lib().hipml_oracle_rng_uniform(C.byref(self._s)))

    def normal(self) -> float:
        return float(lib().hipml_oracle_rng_normal(C.byref(self._s)))

    def normals(self, n: int, std: float = 1.0) -> np.ndarray:
        """n draws of normal_scaled(std), in draw order."""
        out = np.empty(int(n), dtype=np.float32)
        lib().hipml_oracle_rng_fill_normal(C.byref(self._s), C.c_float(std), _p(out, C.c_float),
                                           out.size)
        return out


def attn_causal_f32(q, k_cache, v_cache, n_heads, n_kv, head_dim, seq, scale) -> np.ndarray:
    q, k, v = _f32(q).ravel(), _f32(k_cache).ravel(), _f32(v_cache).ravel()
    out = np.empty(n_heads * head_dim, dtype=np.float32)
    lib().hipml_oracle_attn_causal_f32(_p(q, C.c_float), _p(k, C.c_float), _p(v, C.c_float),
                                       n_heads, n_kv, head_dim, seq, C.c_float(scale),
                                       _p(out, C.c_float))
    return out


def attn_chunk_f32(q, k_cache, v_cache, n_heads, n_kv, head_dim, pos0, tokens, scale,
                   row0: int = 0, row_step: int = 1, threads: int = 1) -> np.ndarray:
    """Chunk prefill: row t = attn_causal_f32 with seq = pos0+t+1. Rows not selected
    by (row0, row_step) are returned as NaN."""
    q, k, v = _f32(q).ravel(), _f32(k_cache).ravel(), _f32(v_cache).ravel()
    out = np.full(tokens * n_heads * head_dim, np.nan, dtype=np.float32)
    lib().hipml_oracle_attn_chunk_f32(_p(q, C.c_float), _p(k, C.c_float), _p(v, C.c_float),
                                      n_heads, n_kv, head_dim, pos0, tokens, C.c_float(scale),
                                      _p(out, C.c_float), row0, row_step, threads)
    return out.reshape(tokens, n_heads * head_dim)


def attn_decode_kv_q8(q, k_bytes, v_bytes, n_heads, n_kv, head_dim, seq, scale,
                      stride: int | None = None) -> np.ndarray:
    q, k, v = _f32(q).ravel(), _u8(k_bytes).ravel(), _u8(v_bytes).ravel()
    stride = seq if stride is None else stride
    row = head_dim // BLOCK * Q8_BLOCK_BYTES
    assert k.size >= n_kv * stride * row and v.size >= n_kv * stride * row
    out = np.empty(n_heads * head_dim, dtype=np.float32)
    lib().hipml_oracle_attn_decode_kv_q8_strided(_p(q, C.c_float), _p(k, C.c_uint8),
                                                 _p(v, C.c_uint8), n_heads, n_kv, head_dim, seq,
                                                 stride, C.c_float(scale), _p(out, C.c_float))
    return out


def attn_decode_f32(q, k, v, n_heads, n_kv, head_dim, seq, scale) -> np.ndarray:
    q, k, v = _f32(q).ravel(), _f32(k).ravel(), _f32(v).ravel()
    out = np.empty(n_heads * head_dim, dtype=np.float32)
    lib().hipml_oracle_attn_decode_f32(_p(q, C.c_float), _p(k, C.c_float), _p(v, C.c_float),
                                       n_heads, n_kv, head_dim, seq, C.c_float(scale),
                                       _p(out, C.c_float))
    return out


def compare(expected, actual) -> tuple[float, float]:
    """parity::compare: (max_abs, max_rel)."""
    e, a = _f32(expected).ravel(), _f32(actual).ravel()
    assert e.size == a.size, f"length mismatch: reference {e.size} vs device {a.size}"
    ma, mr = C.c_float(), C.c_float()
    lib().hipml_oracle_compare(_p(e, C.c_float), _p(a, C.c_float), e.size, C.byref(ma),
                               C.byref(mr))
    return float(ma.value), float(mr.value)


def within(stats: tuple[float, float], tol: tuple[float, float]) -> bool:
    """Stats::within: passes when max_abs <= tol.abs OR max_rel <= tol.rel."""
    return stats[0] <= tol[0] or stats[1] <= tol[1]


TOL_DEFAULT = (1e-4, 1e-3)
TOL_TIGHT = (1e-6, 1e-5)
TOL_EXACT = (0.0, 0.0)


def rel_l2(expected, actual) -> float:
    e = np.asarray(expected, dtype=np.float64).ravel()
    a = np.asarray(actual, dtype=np.float64).ravel()
    return float(np.linalg.norm(e - a) / max(np.linalg.norm(e), 1e-30))


def max_abs(expected, actual) -> float:
    e = np.asarray(expected, dtype=np.float64).ravel()
    a = np.asarray(actual, dtype=np.float64).ravel()
    return float(np.max(np.abs(e - a))) if e.size else 0.0


# ---- attention front end and tail (ops.rs:181-187, 195-224, 260-360) ----------------------

def head_rmsnorm_f32(x, w, n_heads, head_dim, eps) -> np.ndarray:
    x, w = _f32(x), _f32(w)
    out = np.empty(n_heads * head_dim, dtype=np.float32)
    lib().hipml_oracle_head_rmsnorm_f32(_p(x, C.c_float), _p(w, C.c_float), n_heads, head_dim, eps,
                                        _p(out, C.c_float))
    return out


def rope_multi_f32(x, n_heads, head_dim, n_rot, sections, pos, theta_base) -> np.ndarray:
    x = _f32(x)
    out = np.empty(n_heads * head_dim, dtype=np.float32)
    sec = (C.c_int * 4)(*[int(v) for v in sections])
    ps = (C.c_int * 4)(*[int(v) for v in pos])
    lib().hipml_oracle_rope_multi_f32(_p(x, C.c_float), n_heads, head_dim, n_rot, sec, ps,
                                      theta_base, _p(out, C.c_float))
    return out


def rope_neox_f32(x, n_heads, head_dim, pos, theta_base) -> np.ndarray:
    x = _f32(x)
    out = np.empty(n_heads * head_dim, dtype=np.float32)
    lib().hipml_oracle_rope_neox_f32(_p(x, C.c_float), n_heads, head_dim, pos, theta_base,
                                     _p(out, C.c_float))
    return out


def qg_split_f32(qg, n_heads, head_dim):
    """Returns (q, gate), each [n_heads * head_dim]."""
    qg = _f32(qg)
    q = np.empty(n_heads * head_dim, dtype=np.float32)
    gate = np.empty(n_heads * head_dim, dtype=np.float32)
    lib().hipml_oracle_qg_split_f32(_p(qg, C.c_float), n_heads, head_dim, _p(q, C.c_float),
                                    _p(gate, C.c_float))
    return q, gate


def q_gate_f32(q, gate) -> np.ndarray:
    q, gate = _f32(q), _f32(gate)
    out = np.empty(q.size, dtype=np.float32)
    lib().hipml_oracle_q_gate_f32(_p(q, C.c_float), _p(gate, C.c_float), q.size, _p(out, C.c_float))
    return out


def attn_front(qg, k, q_norm, k_norm, n_heads, n_kv, head_dim, n_rot, sections, pos, theta_base,
               eps):
    """The decode front end of attention.rs:117-143 for one token: q|gate split, per-head RMS
    norm of q and k, M-RoPE of both. Returns (q, gate, k)."""
    q, gate = qg_split_f32(qg, n_heads, head_dim)
    q = rope_multi_f32(head_rmsnorm_f32(q, q_norm, n_heads, head_dim, eps), n_heads, head_dim, n_rot,
                       sections, pos, theta_base)
    k = rope_multi_f32(head_rmsnorm_f32(k, k_norm, n_kv, head_dim, eps), n_kv, head_dim, n_rot,
                       sections, pos, theta_base)
    return q, gate, k


# ---- q4_0 (kv.rs:201-218, 238-290, 306-320) -------------------------------------------------

def quantize_q4(values) -> np.ndarray:
    v = _f32(values).ravel()
    assert v.size % BLOCK == 0
    out = np.empty(v.size // BLOCK * Q4_BLOCK_BYTES, dtype=np.uint8)
    lib().hipml_oracle_quantize_q4(_p(v, C.c_float), v.size, _p(out, C.c_uint8))
    return out


def dequantize_q4(data) -> np.ndarray:
    b = _u8(data).ravel()
    assert b.size % Q4_BLOCK_BYTES == 0
    out = np.empty(b.size // Q4_BLOCK_BYTES * BLOCK, dtype=np.float32)
    lib().hipml_oracle_dequantize_q4(_p(b, C.c_uint8), b.size, _p(out, C.c_float))
    return out


def synthetic_blocks_q4(n_blocks: int, seed: int) -> np.ndarray:
    out = np.empty(n_blocks * Q4_BLOCK_BYTES, dtype=np.uint8)
    lib().hipml_oracle_synthetic_blocks_q4(n_blocks, C.c_uint64(seed), _p(out, C.c_uint8))
    return out


def attn_decode_kv(q, k_bytes, v_bytes, dtype, n_heads, n_kv, head_dim, seq, scale,
                   stride: int | None = None) -> np.ndarray:
    """ops::attn_decode_kv over either quantised cache (dtype 0 = q8_0, 1 = q4_0)."""
    q, k, v = _f32(q).ravel(), _u8(k_bytes).ravel(), _u8(v_bytes).ravel()
    stride = seq if stride is None else stride
    row = head_dim // BLOCK * (Q4_BLOCK_BYTES if dtype == 1 else Q8_BLOCK_BYTES)
    assert k.size >= n_kv * stride * row and v.size >= n_kv * stride * row
    out = np.empty(n_heads * head_dim, dtype=np.float32)
    lib().hipml_oracle_attn_decode_kv_strided(_p(q, C.c_float), _p(k, C.c_uint8), _p(v, C.c_uint8),
                                              dtype, n_heads, n_kv, head_dim, seq, stride,
                                              C.c_float(scale), _p(out, C.c_float))
    return out
