"""Thin Python view of the C-ABI launchers, for tests and the bench.

Every function takes CUDA ``torch`` tensors only for their device pointers and the
current stream; the work is done by libhipml_cuda.so. Argument names, order and units
follow the reference's launchers (see include/hipml_cuda.h for the file:line of each).
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib


def _p(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def version() -> str:
    return _lib.load().hipml_version().decode()


def kv_encode(step, k_row, v_row, k_cache, v_cache, n_kv, head_dim, stride, dtype=0):
    """Launcher::kv_encode_ptr_on: quantise one token's K/V rows at step[0]."""
    _lib.check("kv_encode", _lib.load().hipml_kv_encode(
        _stream(), _p(step), dtype, _p(k_row), _p(v_row), _p(k_cache), _p(v_cache), n_kv,
        head_dim, stride))


def kv_encode_bulk(k_f32, v_f32, k_cache, v_cache, n_kv, head_dim, stride, start, src0, rows,
                   dtype=0):
    """Launcher::kv_encode_bulk: rows src0+r of the f32 tile land at position start+r."""
    _lib.check("kv_encode_bulk", _lib.load().hipml_kv_encode_bulk(
        _stream(), dtype, _p(k_f32), _p(v_f32), _p(k_cache), _p(v_cache), n_kv, head_dim, stride,
        start, src0, rows))


def kv_encode_rows(k_f32, v_f32, k_cache, v_cache, n_kv, head_dim, stride, pos, slot_bytes, slots,
                   dtype=0):
    """Launcher::kv_encode_batch: slot s appends its row at pos[2s] in the cache at s*slot_bytes."""
    _lib.check("kv_encode_batch", _lib.load().hipml_kv_encode_rows(
        _stream(), dtype, _p(k_f32), _p(v_f32), _p(k_cache), _p(v_cache), n_kv, head_dim, stride,
        _p(pos), slot_bytes, slots))


def kv_append_f32(step, k_cache, v_cache, k_row, v_row, width):
    _lib.check("kv_append_f32", _lib.load().hipml_kv_append_f32(
        _stream(), _p(step), _p(k_cache), _p(v_cache), _p(k_row), _p(v_row), width))


def kv_append_chunk_f32(k_cache, v_cache, k, v, pos0, width, tokens):
    _lib.check("kv_append_chunk_f32", _lib.load().hipml_kv_append_chunk_f32(
        _stream(), _p(k_cache), _p(v_cache), _p(k), _p(v), pos0, width, tokens))


def attn_decode_kv(step, q, k, v, part_acc, part_ml, out, n_heads, n_kv, head_dim, stride, scale,
                   splits, selector=0, k_off=0, v_off=0):
    """launch_kv::launch_ptrs: split-K decode over the q8 cache + reduce."""
    _lib.check("attn_decode_kv", _lib.load().hipml_attn_decode_kv(
        _stream(), _p(step), selector, _p(q), _p(k), _p(v), _p(part_acc), _p(part_ml), _p(out),
        n_heads, n_kv, head_dim, stride, scale, splits, k_off, v_off))


def attn_decode_cols(pos, q, k, v, part_acc, part_ml, out, n_heads, n_kv, head_dim, stride, scale,
                     splits, cols, acc_slot, ml_slot, q_slot, selector=0):
    """launch_kv::launch_cols_ptrs: `cols` columns of one sequence over a shared cache."""
    _lib.check("attn_decode_cols", _lib.load().hipml_attn_decode_cols(
        _stream(), selector, _p(pos), _p(q), _p(k), _p(v), _p(part_acc), _p(part_ml), _p(out),
        n_heads, n_kv, head_dim, stride, scale, splits, cols, acc_slot, ml_slot, q_slot))


def kv_rows_copy(dst, src, n_kv, row_bytes, dst_stride, src_stride, rows):
    """Live rows [0, rows) of every KV head between two head-major caches (prefix snapshots)."""
    _lib.check("kv_rows_copy", _lib.load().hipml_kv_rows_copy(
        _stream(), _p(dst), _p(src), n_kv, row_bytes, dst_stride, src_stride, rows))


def attn_decode_kv_gated(step, q, k, v, part_acc, part_ml, out, gate, n_heads, n_kv, head_dim,
                         stride, scale, splits, selector=0, k_off=0, v_off=0):
    """attn_decode_kv with out *= sigmoid(gate) applied in the fold."""
    _lib.check("attn_decode_kv_gated", _lib.load().hipml_attn_decode_kv_gated(
        _stream(), _p(step), selector, _p(q), _p(k), _p(v), _p(part_acc), _p(part_ml), _p(out),
        _p(gate), n_heads, n_kv, head_dim, stride, scale, splits, k_off, v_off))


def attn_decode_kv_append(step, k_row, v_row, q, k, v, part_acc, part_ml, out, n_heads, n_kv,
                          head_dim, stride, scale, splits, gate=None, selector=0, k_off=0, v_off=0):
    """One decode step of a layer: append the K/V rows at step[0] (= step[1] - 1), then
    attn_decode_kv (the append is fused into the split pass where that form exists)."""
    _lib.check("attn_decode_kv_append", _lib.load().hipml_attn_decode_kv_append(
        _stream(), _p(step), selector, _p(k_row), _p(v_row), _p(q), _p(k), _p(v), _p(part_acc),
        _p(part_ml), _p(out), _p(gate), n_heads, n_kv, head_dim, stride, scale, splits, k_off, v_off))


def attn_decode_kv_shard(step, q, k, v, part_acc, part_ml, shard_out, n_heads, n_kv, head_dim,
                         stride, scale, splits, selector=0, k_off=0, v_off=0):
    """One GPU's part of a sequence-split decode: writes [n_heads][head_dim+2] =
    (unnormalised acc, max_log2, sum) of the local cache rows."""
    _lib.check("attn_decode_kv_shard", _lib.load().hipml_attn_decode_kv_shard(
        _stream(), _p(step), selector, _p(q), _p(k), _p(v), _p(part_acc), _p(part_ml),
        _p(shard_out), n_heads, n_kv, head_dim, stride, scale, splits, k_off, v_off))


def attn_decode_combine(gathered, out, n_heads, head_dim, shards):
    """Fold the all-gathered shard triples [shards][n_heads][head_dim+2] into out."""
    _lib.check("attn_decode_combine", _lib.load().hipml_attn_decode_combine(
        _stream(), _p(gathered), _p(out), n_heads, head_dim, shards))


def decode_exchange_bytes(n_heads, head_dim, shards) -> int:
    """Bytes of one rank's workspace for attn_decode_kv_shard_exchange (zero it once)."""
    return int(_lib.load().hipml_decode_exchange_bytes(n_heads, head_dim, shards))


def attn_decode_kv_shard_exchange(step, q, k, v, part_acc, part_ml, out, n_heads, n_kv, head_dim,
                                  stride, scale, splits, peer_ws, rank, phases=3,
                                  wait_limit_us=2_000_000, selector=0, k_off=0, v_off=0):
    """Sequence-split decode with the exchange over peer memory: peer_ws = device addresses
    (ints) of every rank's workspace as mapped in this process, peer_ws[rank] the local one."""
    table = (C.c_void_p * len(peer_ws))(*[C.c_void_p(int(a)) for a in peer_ws])
    _lib.check("attn_decode_kv_shard_exchange", _lib.load().hipml_attn_decode_kv_shard_exchange(
        _stream(), _p(step), selector, _p(q), _p(k), _p(v), _p(part_acc), _p(part_ml), _p(out),
        n_heads, n_kv, head_dim, stride, scale, splits, k_off, v_off, table, len(peer_ws), rank,
        phases, wait_limit_us))


def attn_decode_kv_shard_exchange_append(step, k_row, v_row, q, k, v, part_acc, part_ml, out, n_heads,
                                         n_kv, head_dim, stride, scale, splits, peer_ws, rank, phases=3,
                                         wait_limit_us=2_000_000, selector=0, k_off=0, v_off=0):
    """attn_decode_kv_shard_exchange that also appends the token's K/V rows (None on the ranks
    that do not own the new position)."""
    table = (C.c_void_p * len(peer_ws))(*[C.c_void_p(int(a)) for a in peer_ws])
    _lib.check("attn_decode_kv_shard_exchange", _lib.load().hipml_attn_decode_kv_shard_exchange_append(
        _stream(), _p(step), selector, _p(k_row), _p(v_row), _p(q), _p(k), _p(v), _p(part_acc),
        _p(part_ml), _p(out), n_heads, n_kv, head_dim, stride, scale, splits, k_off, v_off, table,
        len(peer_ws), rank, phases, wait_limit_us))


def set_decode_cta_slots(slots: int) -> None:
    _lib.check("set_decode_cta_slots", _lib.load().hipml_set_decode_cta_slots(slots))


def set_decode_fold_mode(mode: int) -> None:
    """0: the split pass folds its own partials (one launch); 1: the fold is a second launch."""
    _lib.check("set_decode_fold_mode", _lib.load().hipml_set_decode_fold_mode(mode))


def set_decode_body(body: int) -> None:
    """1: values on mma.sync (default); 2: values on tcgen05 kind::i8."""
    _lib.check("set_decode_body", _lib.load().hipml_set_decode_body(body))


def decode_plan_quota(lens, splits, n_kv, cta_slots) -> int:
    """64-row tiles per run of the multi-slot decode plan for these live lengths (host mirror)."""
    arr = (C.c_int * len(lens))(*[int(v) for v in lens])
    return int(_lib.load().hipml_decode_plan_quota(arr, len(lens), splits, n_kv, cta_slots))


def attn_decode_kv_static(step, q, k, v, out, n_heads, n_kv, head_dim, stride, scale, splits,
                          selector=0, k_off=0, v_off=0):
    """attn_decode_kv without caller scratch: for callers that cannot allocate device memory.
    The partials live in a 6 MiB array inside the library; calls must not overlap on the GPU."""
    _lib.check("attn_decode_kv_static", _lib.load().hipml_attn_decode_kv_static(
        _stream(), _p(step), selector, _p(q), _p(k), _p(v), _p(out), n_heads, n_kv, head_dim,
        stride, scale, splits, k_off, v_off))


def attn_decode_cols_f32(q, k_cache, v_cache, part_acc, part_ml, out, n_heads, n_kv, head_dim,
                         n_ctx, pos0, rows):
    """AttnLayer::attention_cols: f32-cache decode of `rows` consecutive columns."""
    _lib.check("attention_cols", _lib.load().hipml_attn_decode_cols_f32(
        _stream(), _p(q), _p(k_cache), _p(v_cache), _p(part_acc), _p(part_ml), _p(out), n_heads,
        n_kv, head_dim, n_ctx, pos0, rows))


def kv_append_cols_f32(k_cache, v_cache, k, v, pos0, rows, width):
    """AttnLayer::append_rows."""
    _lib.check("kv_append_cols_f32", _lib.load().hipml_kv_append_cols_f32(
        _stream(), _p(k_cache), _p(v_cache), _p(k), _p(v), pos0, rows, width))


def cols_splits(n_ctx: int) -> int:
    """split_geom (crates/hipml-kernels/src/attn_gpu/imp/attn_cols.rs:15-20)."""
    return min(max((n_ctx + 31) // 32, 1), 64)


def attn_decode_rows(pos, q, k_cache, v_cache, part_acc, part_ml, out, n_heads, n_kv, head_dim,
                     stride, scale, splits, kv_slot_bytes, acc_slot, ml_slot, q_slot, slots,
                     dtype=0):
    """Launcher::attn_decode_rows_ptr: multi-slot decode, runs fixed in cache positions."""
    _lib.check("attn_decode_rows", _lib.load().hipml_attn_decode_rows(
        _stream(), dtype, _p(pos), _p(q), _p(k_cache), _p(v_cache), _p(part_acc), _p(part_ml),
        _p(out), n_heads, n_kv, head_dim, stride, scale, splits, kv_slot_bytes, acc_slot, ml_slot,
        q_slot, slots))


def attn_decode_batch(pos, q, k_cache, v_cache, part_acc, part_ml, out, n_heads, n_kv, head_dim,
                      stride, scale, splits, kv_slot_bytes, acc_slot, ml_slot, q_slot, slots,
                      live_seq, dtype=0):
    """Launcher::attn_decode_batch."""
    _lib.check("attn_decode_batch", _lib.load().hipml_attn_decode_batch(
        _stream(), dtype, _p(pos), _p(q), _p(k_cache), _p(v_cache), _p(part_acc), _p(part_ml),
        _p(out), n_heads, n_kv, head_dim, stride, scale, splits, kv_slot_bytes, acc_slot, ml_slot,
        q_slot, slots, live_seq))


def attn_decode_batch_append(pos, k_f32, v_f32, q, k_cache, v_cache, part_acc, part_ml, out, n_heads,
                             n_kv, head_dim, stride, scale, splits, kv_slot_bytes, acc_slot, ml_slot,
                             q_slot, slots, dtype=0):
    """One batched decode step of a layer: kv_encode_rows + attn_decode_rows, the append fused
    into the split pass where that form exists."""
    _lib.check("attn_decode_batch_append", _lib.load().hipml_attn_decode_batch_append(
        _stream(), dtype, _p(pos), _p(k_f32), _p(v_f32), _p(q), _p(k_cache), _p(v_cache),
        _p(part_acc), _p(part_ml), _p(out), n_heads, n_kv, head_dim, stride, scale, splits,
        kv_slot_bytes, acc_slot, ml_slot, q_slot, slots))


def attn_chunk_workspace_bytes(n_kv, head_dim, pos0, tokens) -> int:
    return int(_lib.load().hipml_attn_chunk_workspace_bytes(n_kv, head_dim, pos0, tokens))


def attn_chunk(q, k_cache, v_cache, out, n_heads, n_kv, head_dim, pos0, tokens, kv_dtype=0,
               stride=0, part_acc=None, part_ml=None, splits=1, mode=0, workspace=None):
    """AttnLayer::chunk_attention / chunk_attention_q8 / chunk_attention_q8_split."""
    ws_bytes = 0 if workspace is None else workspace.numel() * workspace.element_size()
    _lib.check("chunk_attention", _lib.load().hipml_attn_chunk(
        _stream(), _p(q), _p(k_cache), _p(v_cache), _p(out), n_heads, n_kv, head_dim, pos0,
        tokens, kv_dtype, stride, _p(part_acc), _p(part_ml), splits, mode, _p(workspace),
        ws_bytes))


def attn_chunk_stage(k_cache, v_cache, n_kv, head_dim, kv_dtype, stride, key_from, key_to,
                     key_capacity, workspace):
    """Convert cache rows [key_from, key_to) into the tensor-core operand image."""
    _lib.check("chunk_attention stage", _lib.load().hipml_attn_chunk_stage(
        _stream(), _p(k_cache), _p(v_cache), n_kv, head_dim, kv_dtype, stride, key_from, key_to,
        key_capacity, _p(workspace), workspace.numel() * workspace.element_size()))


def attn_chunk_staged(q, out, n_heads, n_kv, head_dim, pos0, tokens, key_capacity, workspace,
                      part_acc=None, part_ml=None, splits=1, mode=0):
    """Chunk attention over rows already staged by attn_chunk_stage."""
    _lib.check("chunk_attention", _lib.load().hipml_attn_chunk_staged(
        _stream(), _p(q), _p(out), n_heads, n_kv, head_dim, pos0, tokens, _p(part_acc),
        _p(part_ml), splits, mode, key_capacity, _p(workspace),
        workspace.numel() * workspace.element_size()))


# ---- attention front end and tail -----------------------------------------------------------

def _sections(sections):
    return None if sections is None else (C.c_int * 4)(*[int(v) for v in sections])


def attn_front(qg, q, gate, k, q_norm, k_norm, n_heads, n_kv, head_dim, n_rot, sections, pos,
               theta_base, eps):
    """AttnLayer::front: one token, q|gate split + head RMS norm + M-RoPE (k in place)."""
    _lib.check("attn_front", _lib.load().hipml_attn_front(
        _stream(), _p(qg), _p(q), _p(gate), _p(k), _p(q_norm), _p(k_norm), n_heads, n_kv, head_dim,
        n_rot, _sections(sections), _p(pos), theta_base, eps))


def qg_split_chunk(qg, q, gate, n_heads, head_dim, tokens):
    _lib.check("qg_split_chunk", _lib.load().hipml_qg_split_chunk(
        _stream(), _p(qg), _p(q), _p(gate), n_heads, head_dim, tokens))


def norm_rope_chunk(q, k, q_norm, k_norm, n_heads, n_kv, head_dim, n_rot, theta_base, eps, pos0,
                    tokens):
    _lib.check("norm_rope_chunk", _lib.load().hipml_norm_rope_chunk(
        _stream(), _p(q), _p(k), _p(q_norm), _p(k_norm), n_heads, n_kv, head_dim, n_rot, theta_base,
        eps, pos0, tokens))


def q_gate(q, gate, y, n):
    _lib.check("q_gate", _lib.load().hipml_q_gate(_stream(), _p(q), _p(gate), _p(y), n))


def attn_front_append_q8(qg, k, v, q, gate, q_norm, k_norm, k_cache, v_cache, n_heads, n_kv,
                         head_dim, n_rot, theta_base, eps, pos0=0, tokens=1, stride=0, sections=None,
                         pos=None, step=None, k_out=None):
    """Split + norm + rope + q8_0 append of `tokens` rows in one launch."""
    _lib.check("attn_front_append_q8", _lib.load().hipml_attn_front_append_q8(
        _stream(), _p(qg), _p(k), _p(v), _p(q), _p(gate), _p(k_out), _p(q_norm), _p(k_norm),
        _p(k_cache), _p(v_cache), n_heads, n_kv, head_dim, n_rot, _sections(sections), _p(pos),
        _p(step), pos0, tokens, stride, theta_base, eps))


def attn_chunk_staged_gated(q, out, gate, n_heads, n_kv, head_dim, pos0, tokens, key_capacity,
                            workspace, part_acc=None, part_ml=None, splits=1, mode=0):
    """attn_chunk_staged with out *= sigmoid(gate) applied in the epilogue / combine."""
    _lib.check("chunk_attention", _lib.load().hipml_attn_chunk_staged_gated(
        _stream(), _p(q), _p(out), _p(gate), n_heads, n_kv, head_dim, pos0, tokens, _p(part_acc),
        _p(part_ml), splits, mode, key_capacity, _p(workspace),
        workspace.numel() * workspace.element_size()))


def check_device_status() -> int:
    """Synchronises the current stream; raises if a kernel's bounded wait ran out."""
    st = C.c_int(0)
    _lib.check("device status", _lib.load().hipml_check_device_status(_stream(), C.byref(st)))
    return st.value


# ---- split policies (host arithmetic of the reference's engine) -------------------------

def decode_splits(seq: int) -> int:
    """DeepKv::splits for the warp-kernel family (crates/hipml-model/src/gpu/deep_kv.rs:102-110)."""
    fine = min(max(seq // 8, 1), 128)
    coarse = min(max(seq // 64, 1), 256)
    return max(fine, coarse)


def batch_splits(stride: int, slots: int) -> int:
    """attn_splits (crates/hipml-model/src/gpu/batch/kv.rs:39-42)."""
    per = 64 * max((slots + 3) // 4, 1)
    return min(max((stride + per - 1) // per, 1), 256)


def prefill_splits(pos0: int, configured: int = 8, split_min: int = 8192) -> int:
    """split_count (crates/hipml-model/src/gpu/attn_tile.rs:138-151)."""
    return configured if pos0 >= split_min else 1
