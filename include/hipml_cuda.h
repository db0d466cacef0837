/*
 * hipml_cuda.h -- C ABI of libhipml_cuda.so: the B200 (sm_100a) replacement for
 * hipml's device layer and its full-attention kernel launchers.
 *
 * Two groups of entry points:
 *
 *   A. Device layer. One flat function per symbol of the reference's vendor
 *      binding (crates/hipml-hip/src/ffi.rs:29-105), same argument order and
 *      the same conventions: every call returns an int, 0 is success, handles
 *      are opaque pointers, memcpy kinds are 1 = host->device, 2 = device->host,
 *      3 = device->device. A `hipml-cuda` crate binds these 1:1 where
 *      `hipml-hip` binds amdhip64.
 *
 *   B. Attention launchers. One function per launch routine of the
 *      reference's kernel crate for the full-attention path (KV append /
 *      quantise, split-K decode over the q8_0 cache, multi-slot decode, causal
 *      chunk prefill). Arguments keep the reference's order, units and
 *      meaning; grid/block geometry, shared-memory sizes and tensor-map setup
 *      are internal. All pointers are device pointers unless stated; `stream`
 *      is a CUDA stream handle (NULL = the default stream); launches are
 *      asynchronous on that stream.
 *
 * Errors: 0 = success. Codes 1..9999 are CUDA runtime error codes. Codes
 * >= HIPML_ERR_BASE are argument errors raised by this library before
 * anything is launched; hipml_last_error_message() then holds the same
 * sentence the reference's launcher returns as Err(String).
 *
 * Cache layout (frozen by the reference, crates/hipml-core/src/kv.rs:22-44):
 * q8_0 block = f16 scale (LE) + 32 int8 codes = 34 bytes; block (kvh, pos, c)
 * at byte ((kvh*stride + pos)*(head_dim/32) + c)*34; K and V are separate
 * arrays; slot b of a batched cache starts at b*slot_bytes. The f32 cache is
 * position-major [n_ctx][n_kv*head_dim].
 */
#ifndef HIPML_CUDA_H
#define HIPML_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void *hipml_stream_t;
typedef void *hipml_event_t;
typedef void *hipml_graph_t;
typedef void *hipml_graph_exec_t;
typedef void *hipml_module_t;
typedef void *hipml_function_t;

#define HIPML_SUCCESS 0
#define HIPML_ERR_BASE 10000
#define HIPML_ERR_INVALID_ARGUMENT 10001 /* shape / dtype / alignment rejected */
#define HIPML_ERR_UNKNOWN_KERNEL 10002   /* module lookup by name failed */
#define HIPML_ERR_WORKSPACE 10003        /* workspace missing or too small */
#define HIPML_ERR_DEVICE_STATUS 10004    /* a kernel reported a bounded-wait timeout */

#define HIPML_MEMCPY_HOST_TO_DEVICE 1
#define HIPML_MEMCPY_DEVICE_TO_HOST 2
#define HIPML_MEMCPY_DEVICE_TO_DEVICE 3

/* ------------------------------------------------------------------ A. device
 * Each replaces the hip* symbol of the same name in
 * crates/hipml-hip/src/ffi.rs (line given). */

int hipml_init(unsigned flags);                                           /* ffi.rs:30 hipInit */
int hipml_get_device_count(int *count);                                   /* ffi.rs:31 */
int hipml_get_device(int *device, int ordinal);                           /* ffi.rs:32 */
int hipml_set_device(int device);                                         /* ffi.rs:33 */
int hipml_device_get_name(char *name, int len, int device);               /* ffi.rs:34 */
int hipml_device_total_mem(size_t *bytes, int device);                    /* ffi.rs:35 */
int hipml_device_compute_capability(int *major, int *minor, int device);  /* ffi.rs:36-40 */
const char *hipml_get_error_string(int code);                             /* ffi.rs:41 */
/* Detail of the last HIPML_ERR_* raised on the calling thread ("" if none). */
const char *hipml_last_error_message(void);

int hipml_malloc(void **ptr, size_t size);                                /* ffi.rs:43 */
int hipml_free(void *ptr);                                                /* ffi.rs:44 */
int hipml_memset(void *dst, int value, size_t size);                      /* ffi.rs:45 */
int hipml_mem_get_info(size_t *free_bytes, size_t *total_bytes);          /* ffi.rs:46 */
int hipml_memcpy(void *dst, const void *src, size_t size, int kind);      /* ffi.rs:47 */
int hipml_memcpy_async(void *dst, const void *src, size_t size, int kind,
                       hipml_stream_t stream);                            /* ffi.rs:76-82 */
int hipml_device_synchronize(void);                                       /* ffi.rs:48 */
/* Pinned host memory for the asynchronous copies (no counterpart in ffi.rs:
 * the reference uploads from pageable memory). */
int hipml_host_alloc(void **ptr, size_t size);
int hipml_host_free(void *ptr);

int hipml_event_create(hipml_event_t *event);                             /* ffi.rs:50 */
int hipml_event_destroy(hipml_event_t event);                             /* ffi.rs:51 */
int hipml_event_record(hipml_event_t event, hipml_stream_t stream);       /* ffi.rs:52 */
int hipml_event_synchronize(hipml_event_t event);                         /* ffi.rs:53 */
int hipml_event_elapsed_time(float *ms, hipml_event_t start, hipml_event_t stop); /* ffi.rs:54 */

int hipml_stream_create(hipml_stream_t *stream);                          /* ffi.rs:56 */
int hipml_stream_destroy(hipml_stream_t stream);                          /* ffi.rs:57 */
int hipml_stream_synchronize(hipml_stream_t stream);                      /* ffi.rs:58 */
int hipml_stream_wait_event(hipml_stream_t stream, hipml_event_t event, unsigned flags); /* ffi.rs:59 */

int hipml_stream_begin_capture(hipml_stream_t stream, int mode);          /* ffi.rs:63 (0 = global) */
int hipml_stream_end_capture(hipml_stream_t stream, hipml_graph_t *graph);/* ffi.rs:64 */
int hipml_graph_instantiate(hipml_graph_exec_t *exec, hipml_graph_t graph, void *error_node,
                            char *log_buffer, size_t log_size);           /* ffi.rs:65-71 */
int hipml_graph_launch(hipml_graph_exec_t exec, hipml_stream_t stream);   /* ffi.rs:72 */
int hipml_graph_upload(hipml_graph_exec_t exec, hipml_stream_t stream);   /* ffi.rs:73 */
int hipml_graph_destroy(hipml_graph_t graph);                             /* ffi.rs:74 */
int hipml_graph_exec_destroy(hipml_graph_exec_t exec);                    /* ffi.rs:75 */

/* The kernels are linked into this library, so there is one built-in module;
 * `file` is accepted for signature compatibility and may be NULL.
 * hipml_module_get_function resolves the reference's kernel entry names
 * (kv_encode_q8, kv_encode_bulk_q8, kv_encode_q8_b, kv_append_f32,
 * kv_append_chunk_f32, attn_decode_kv_reduce, attn_decode_kv_reduce_b); those
 * keep the reference's parameter lists and launch shapes, so
 * hipml_module_launch_kernel(f, grid, block, shmem, stream, params, NULL)
 * launches them exactly as `Kernel::launch` does
 * (crates/hipml-hip/src/device.rs:543-580). The attention kernels proper need
 * launch state that a bare parameter array cannot carry; use section B. */
int hipml_module_load(hipml_module_t *module, const char *file);          /* ffi.rs:84 */
int hipml_module_unload(hipml_module_t module);                           /* ffi.rs:85 */
int hipml_module_get_function(hipml_function_t *function, hipml_module_t module,
                              const char *name);                          /* ffi.rs:86-90 */
int hipml_module_launch_kernel(hipml_function_t function, unsigned grid_x, unsigned grid_y,
                               unsigned grid_z, unsigned block_x, unsigned block_y,
                               unsigned block_z, unsigned shared_mem_bytes, hipml_stream_t stream,
                               void **kernel_params, void **extra);       /* ffi.rs:91-104 */

/* --------------------------------------------------------------- B. launchers
 * `dtype` for encode/decode is KvDtype::id(): 0 = q8_0 (34-byte blocks), 1 = q4_0
 * (18-byte blocks, crates/hipml-core/src/kv.rs:36-90). `step` is the device-resident i32[8] step buffer
 * [pos, seq, token, 0, p0..p3] (crates/hipml-kernels/src/launch.rs:105-154):
 * step[0] = append position, step[1] = live length. */

/* Launcher::kv_encode_ptr_on (crates/hipml-kernels/src/launch/device/graph_launch.rs:932-973):
 * quantise one token's K and V rows ([n_kv*head_dim] f32 each) into the cache at step[0]. */
int hipml_kv_encode(hipml_stream_t stream, const int *step, int dtype, const float *k_row,
                    const float *v_row, void *k_cache, void *v_cache, int n_kv, int head_dim,
                    int stride);

/* Launcher::kv_encode_bulk (graph_launch.rs:980-1028): `rows` positions of a
 * position-major [.][n_kv*head_dim] f32 buffer; source row src0+r lands at position start+r. */
int hipml_kv_encode_bulk(hipml_stream_t stream, int dtype, const float *k_f32, const float *v_f32,
                         void *k_cache, void *v_cache, int n_kv, int head_dim, int stride,
                         int start, int src0, int rows);

/* Launcher::kv_encode_rows_ptr / kv_encode_batch
 * (crates/hipml-kernels/src/launch/device/batch_launch.rs:22-105): one row per slot, slot s
 * appends at pos[2*s] into the cache at byte s*slot_bytes. pos is i32 [slots][2] = (pos, pos+1). */
int hipml_kv_encode_rows(hipml_stream_t stream, int dtype, const float *k_f32, const float *v_f32,
                         void *k_cache, void *v_cache, int n_kv, int head_dim, int stride,
                         const int *pos, int slot_bytes, int slots);

/* AttnLayer::append_at (crates/hipml-kernels/src/attn_gpu.rs:885-912; kernel
 * kv_append_f32.hip:10-26): copy one K and one V row into the f32 caches at step[0]. */
int hipml_kv_append_f32(hipml_stream_t stream, const int *step, float *k_cache, float *v_cache,
                        const float *k_row, const float *v_row, int width);

/* kv_append_chunk_f32 (crates/hipml-kernels/kernels/attn_chunk_f32.hip:100-119): rows
 * t < tokens of k/v land at cache row pos0+t. */
int hipml_kv_append_chunk_f32(hipml_stream_t stream, float *k_cache, float *v_cache,
                              const float *k, const float *v, int pos0, int width, int tokens);

/* launch_kv::launch_ptrs (crates/hipml-kernels/src/launch_kv.rs:110-280): split-K decode over
 * the q8_0 cache and the fold of the split partials into out f32 [n_heads][head_dim].
 * `selector` is the reference's kernel id: 0 and 4 select the tensor-core kernel (head_dim 256
 * only), 1 the same kernel over a q4_0 cache, 6 the scalar kernel (any head_dim in 32..256
 * step 32); other ids are rejected. `stride` is the cache's rows per KV head; the live length
 * is step[1]. k_off/v_off are byte offsets (multiples of 16) added to k/v.
 * part_acc f32 [n_heads][splits][head_dim] and part_ml f32 [n_heads][splits][2] = (max in log2
 * units, sum) are SCRATCH: only `out` is defined. The reference makes two launches (split pass,
 * attn_decode_kv_reduce, launch_kv.rs:232-279) with split s over positions [s*per, (s+1)*per),
 * per = ceil(seq/splits). The scalar kernel (selector 6, or any head_dim other than 256) keeps
 * exactly that and fills every slot. The tensor-core kernel is ONE launch and deals the rows
 * out for this device instead: R = max(1, min(splits, ceil(seq/64), CTA slots / n_kv)) runs
 * per KV head, balanced to within one 64-row tile, partial of run r in slot r; slots from R up
 * to min(splits, CTA slots / n_kv) receive neutral partials (max -inf, sum 0), slots past that
 * are not written at all; the CTA that completes a group of eight runs folds it into the
 * group's first slot, and the last CTA of a KV head folds the groups and writes `out`. A
 * caller must therefore not point the by-name attn_decode_kv_reduce kernel at these partials.
 * The tensor-core kernel needs out, part_acc (16 bytes) and part_ml (8 bytes) aligned. Two
 * calls that may overlap on the device must not share scratch (as in the reference); the
 * arrival counters of the in-kernel fold are library memory, keyed by stream (and capture),
 * and need no care from the caller. */
int hipml_attn_decode_kv(hipml_stream_t stream, const int *step, int selector, const float *q,
                         const void *k, const void *v, float *part_acc, float *part_ml,
                         float *out, int n_heads, int n_kv, int head_dim, int stride, float scale,
                         int splits, size_t k_off, size_t v_off);

/* AttnLayer::attention_cols (crates/hipml-kernels/src/attn_gpu/imp/attn_cols.rs:66-173): split-K
 * decode over the f32 position-major cache [n_ctx][n_kv*head_dim] for `rows` consecutive
 * columns; column c is the query at position pos0 + c and sees cache rows 0..pos0+c. q and out
 * are f32 [rows][n_heads*head_dim]. The key axis is cut into splits = clamp(ceil(n_ctx/32), 1,
 * 64) runs of ceil(n_ctx/splits) rows fixed in cache positions (split_geom, attn_cols.rs:15-20);
 * part_acc is f32 [rows][n_heads][splits][head_dim], part_ml f32 [rows][n_heads][splits][2]
 * (split_scratch, attn_cols.rs:24-31). scale is 1/sqrt(head_dim). */
int hipml_attn_decode_cols_f32(hipml_stream_t stream, const float *q, const float *k_cache,
                               const float *v_cache, float *part_acc, float *part_ml, float *out,
                               int n_heads, int n_kv, int head_dim, int n_ctx, int pos0,
                               int rows);

/* AttnLayer::append_rows (attn_cols.rs:34-64; kernel kv_append_cols_f32.hip:11-31): row c of
 * k/v ([rows][width] f32) lands at cache row pos0 + c. */
int hipml_kv_append_cols_f32(hipml_stream_t stream, float *k_cache, float *v_cache,
                             const float *k, const float *v, int pos0, int rows, int width);

/* launch_kv::launch_cols_ptrs as used by deep_attention_cols (crates/hipml-model/src/gpu/
 * attn_tile.rs:225-295): decode of `cols` consecutive columns of ONE sequence (speculative
 * verify). The columns share the cache; column c has its own query row (q + c*q_slot floats),
 * (position, length) pair (pos[2c], pos[2c+1]), scratch slices (c*acc_slot, c*ml_slot floats)
 * and output row (out + c*q_slot). Every column is partitioned over its own live length with
 * the given split count, so its result is bit-identical to its one-column hipml_attn_decode_kv
 * launch (the caller groups columns of equal split count, as the reference does). selector 0
 * or 4. */
int hipml_attn_decode_cols(hipml_stream_t stream, int selector, const int *pos, const float *q,
                           const void *k, const void *v, float *part_acc, float *part_ml,
                           float *out, int n_heads, int n_kv, int head_dim, int stride, float scale,
                           int splits, int cols, int acc_slot, int ml_slot, int q_slot);

/* The attention half of a prefix snapshot / restore (crates/hipml-model/src/gpu/prefix.rs:30-43
 * copies the whole head-major buffer): only the live rows [0, rows) of every KV head move,
 * between a cache with `src_stride` rows per head and one with `dst_stride` (a snapshot sized
 * for the prefix has dst_stride = rows). row_bytes = 272 for q8_0 at head_dim 256. */
int hipml_kv_rows_copy(hipml_stream_t stream, void *dst, const void *src, int n_kv, int row_bytes,
                       int dst_stride, int src_stride, int rows);

/* hipml_attn_decode_kv with the layer's output gate applied where the output row is produced:
 * out = attention * sigmoid(gate), gate f32 [n_heads][head_dim] (no counterpart as one call in
 * the reference, which launches q_gate_f32 after the reduce, attn_gpu.rs:798-830). */
int hipml_attn_decode_kv_gated(hipml_stream_t stream, const int *step, int selector, const float *q,
                               const void *k, const void *v, float *part_acc, float *part_ml,
                               float *out, const float *gate, int n_heads, int n_kv, int head_dim,
                               int stride, float scale, int splits, size_t k_off, size_t v_off);

/* One decode step of a layer in one call: append the token's K/V rows (f32 [n_kv][head_dim]) at
 * step[0], then hipml_attn_decode_kv over the step[1] live rows (the reference makes the two
 * launches kv_encode_ptr_on + launch_ptrs, crates/hipml-model/src/gpu/attn_tile.rs:150-224).
 * step[0] must be step[1] - 1 (device status 22 otherwise). With selector 0 / 1 / 4, head_dim 256
 * and 16-byte aligned rows and caches the append happens inside the split pass -- the CTA
 * whose run ends the sequence quantises the row into its tile and stores it to the cache,
 * bit-identical to hipml_kv_encode -- otherwise the two launches are made here. `gate` is
 * optional (NULL: none) and applied as in hipml_attn_decode_kv_gated. */
int hipml_attn_decode_kv_append(hipml_stream_t stream, const int *step, int selector,
                                const float *k_row, const float *v_row, const float *q, void *k,
                                void *v, float *part_acc, float *part_ml, float *out,
                                const float *gate, int n_heads, int n_kv, int head_dim, int stride,
                                float scale, int splits, size_t k_off, size_t v_off);

/* One batched decode step of a layer in one call: hipml_kv_encode_rows (slot s appends row
 * k_f32 + s*n_kv*head_dim at pos[2s], which must be pos[2s+1] - 1) then hipml_attn_decode_rows;
 * with dtype 0 / 1, head_dim 256 and 16-byte aligned buffers the append happens inside the split
 * pass, otherwise the two launches are made here. */
int hipml_attn_decode_batch_append(hipml_stream_t stream, int dtype, const int *pos,
                                   const float *k_f32, const float *v_f32, const float *q,
                                   void *k_cache, void *v_cache, float *part_acc, float *part_ml,
                                   float *out, int n_heads, int n_kv, int head_dim, int stride,
                                   float scale, int splits, int kv_slot_bytes, int acc_slot,
                                   int ml_slot, int q_slot, int slots);

/* ---- Attention front end and tail (the callers either side of the attention kernels) ----
 * CPU definition: crates/hipml-core/src/ops.rs:181-187, 260-360, composed as in
 * attention.rs:117-143. q|gate rows are [n_heads][2*head_dim] (q half first), q / gate rows
 * [n_heads][head_dim], k rows [n_kv][head_dim]; M-RoPE rotates the first n_rot channels (NeoX
 * pairs c, c + n_rot/2; frequency theta_base^(-2c/n_rot); f64 angles); sections[4] chooses
 * which of the four position ids feeds pair c (NULL or all 0: id 0 for every pair). */

/* AttnLayer::front (crates/hipml-kernels/src/attn_gpu.rs:552-600; kernel attn_front_f32.hip:
 * 34-135): one token. q|gate split, RMS norm of q (weights q_norm) and of k in place
 * (k_norm), M-RoPE of both; pos = device int[4]. */
int hipml_attn_front(hipml_stream_t stream, const float *qg, float *q, float *gate, float *k,
                     const float *q_norm, const float *k_norm, int n_heads, int n_kv, int head_dim,
                     int n_rot, const int *sections, const int *pos, float theta_base, float eps);

/* The chunk forms (crates/hipml-kernels/src/attn_gpu/imp/attn_chunk.rs:145-199; kernels
 * attn_chunk_f32.hip:22-98): rows of `tokens` tokens, text positions pos0 + t. */
int hipml_qg_split_chunk(hipml_stream_t stream, const float *qg, float *q, float *gate, int n_heads,
                         int head_dim, int tokens);
int hipml_norm_rope_chunk(hipml_stream_t stream, float *q, float *k, const float *q_norm,
                          const float *k_norm, int n_heads, int n_kv, int head_dim, int n_rot,
                          float theta_base, float eps, int pos0, int tokens);

/* The output gate, y = q * sigmoid(gate) over n elements, y may alias q (attn_chunk.rs:345-362;
 * kernel q_gate_f32.hip). */
int hipml_q_gate(hipml_stream_t stream, const float *q, const float *gate, float *y, long long n);

/* All of the front end in one pass, with the q8_0 append (no counterpart in the reference,
 * which runs split, norm+rope and kv_encode as separate launches): for every token t the q|gate
 * row is split, q and k are normalised and rotated, and the rotated k row and the v row are
 * quantised straight into cache row pos0 + t. head_dim 256, n_rot a multiple of 16.
 * k_out (optional) receives the rotated k rows as f32; k_cache / v_cache may both be NULL (no
 * append). For one decode token give pos (device int[4], M-RoPE ids) and / or step (device,
 * step[0] = cache row) instead of pos0. */
int hipml_attn_front_append_q8(hipml_stream_t stream, const float *qg, const float *k,
                               const float *v, float *q, float *gate, float *k_out,
                               const float *q_norm, const float *k_norm, void *k_cache,
                               void *v_cache, int n_heads, int n_kv, int head_dim, int n_rot,
                               const int *sections, const int *pos, const int *step, int pos0,
                               int tokens, int stride, float theta_base, float eps);

/* Sequence-split decode across GPUs (no counterpart in the reference, which is single-GPU; the
 * algebra is its split-K reduce, crates/hipml-kernels/kernels/attn_decode_kv.hip:491-532, lifted
 * from thread blocks to devices). Each GPU holds a contiguous range of every KV head's positions
 * in its own cache and runs hipml_attn_decode_kv_shard: same arguments as hipml_attn_decode_kv
 * (step[1] = the live length of the LOCAL cache, 0 allowed), but instead of the normalised
 * output it writes the folded triple of its shard: shard_out f32 [n_heads][head_dim + 2] =
 * (unnormalised acc[head_dim], max in log2 units, sum). The shards' rows are exchanged with any
 * all-gather (NCCL) into gathered f32 [shards][n_heads][head_dim + 2], and
 * hipml_attn_decode_combine folds them into out f32 [n_heads][head_dim]. */
int hipml_attn_decode_kv_shard(hipml_stream_t stream, const int *step, int selector,
                               const float *q, const void *k, const void *v, float *part_acc,
                               float *part_ml, float *shard_out, int n_heads, int n_kv,
                               int head_dim, int stride, float scale, int splits, size_t k_off,
                               size_t v_off);
int hipml_attn_decode_combine(hipml_stream_t stream, const float *gathered, float *out,
                              int n_heads, int head_dim, int shards);

/* The same sequence-split decode with the exchange done by the decode kernel itself over peer
 * memory instead of a collective call (no counterpart in the reference). Every rank owns a
 * workspace of hipml_decode_exchange_bytes(...) bytes, 256-byte aligned, zero-filled once
 * before the first call, that every other rank has mapped (peer access, IPC handle or
 * symmetric memory); peer_ws is a HOST array of `shards` device pointers, peer_ws[w] = rank w's
 * workspace as mapped in this process, peer_ws[rank] = the local one. One call: the split
 * pass over the local rows, whose last CTA per KV head folds the local partials, stores the
 * folded triples into every rank's workspace (each value tagged with the call's number in the
 * same 64-bit store), waits until every rank's values of the same call have arrived and folds
 * the shards into out f32 [n_heads][head_dim] - ONE launch up to 2 ranks; with more, the
 * split pass leaves its triples in the workspace's staging rows and a second launch of
 * (head, rank) CTAs does the stores and the collect (one SM cannot feed NVLink for many
 * peers). head_dim 256, selectors 0, 1, 4. All ranks must make the same sequence of calls. phases: 3 = all of it; 1 = split pass +
 * publish only and 2 = wait + final fold only, a small launch of its own (the two halves, for
 * hosts that drive several ranks from one stream). Adding 4 to phases divides the result by
 * head (n_heads must be a multiple of shards): head h's triples go only to rank
 * h / (n_heads / shards), which alone folds them and writes row h of `out`; a rank's other rows
 * of `out` are left as they were. That is the input layout of a row-parallel output
 * projection, every triple crosses NVLink once instead of `shards` times, and the call stays
 * one launch at any rank count. The wait is bounded in time by
 * wait_limit_us (capped at 10 s): when it runs out the kernel leaves `out` untouched and
 * hipml_check_device_status reports 31. If a rank misses a call the ranks' call numbers
 * differ for good: zero every rank's workspace (between steps, with a host barrier) to
 * resynchronise. Safe to capture in a graph and replay (the call counters live in the
 * workspace and only grow). The _append form also appends the token's K/V rows (as
 * hipml_attn_decode_kv_append) on the rank that owns the new position; pass NULL rows on the
 * others. */
size_t hipml_decode_exchange_bytes(int n_heads, int head_dim, int shards);
int hipml_attn_decode_kv_shard_exchange(hipml_stream_t stream, const int *step, int selector,
                                        const float *q, const void *k, const void *v,
                                        float *part_acc, float *part_ml, float *out, int n_heads,
                                        int n_kv, int head_dim, int stride, float scale, int splits,
                                        size_t k_off, size_t v_off, void *const *peer_ws,
                                        int shards, int rank, int phases,
                                        unsigned wait_limit_us);
int hipml_attn_decode_kv_shard_exchange_append(hipml_stream_t stream, const int *step, int selector,
                                               const float *k_row, const float *v_row,
                                               const float *q, void *k, void *v, float *part_acc,
                                               float *part_ml, float *out, int n_heads, int n_kv,
                                               int head_dim, int stride, float scale, int splits,
                                               size_t k_off, size_t v_off, void *const *peer_ws,
                                               int shards, int rank, int phases,
                                               unsigned wait_limit_us);

/* The same decode for callers that cannot allocate device memory (this entry has no
 * counterpart in the reference): a host that serves from a fixed arena and may not call
 * cudaMalloc, a binding without a device allocator, a loop that must stay clear of the
 * allocator. The split partials live in a device array inside the library image (6.05 MiB,
 * held by every GPU that loads the library until the process exits) instead of caller
 * buffers; inputs and the output are still the caller's. Limit: n_heads * splits *
 * (head_dim + 2) <= 24 * 256 * 258 floats, otherwise HIPML_ERR_WORKSPACE and nothing runs.
 * The first call on a device looks up the array's device address; make it before any stream
 * capture. All calls share the array (it keeps the previous call's partials; nothing needs
 * clearing because every slot that is folded is written first), so calls that overlap on the
 * GPU race: keep them ordered on one stream or with events. No allocation is made here. */
int hipml_attn_decode_kv_static(hipml_stream_t stream, const int *step, int selector,
                                const float *q, const void *k, const void *v, float *out,
                                int n_heads, int n_kv, int head_dim, int stride, float scale,
                                int splits, size_t k_off, size_t v_off);

/* Launcher::attn_decode_rows_ptr (batch_launch.rs:213-316): multi-slot decode. Slot s reads
 * q + s*q_slot, caches + s*kv_slot_bytes, pos[2*s+1] as its live length, and writes
 * part_acc + s*acc_slot, part_ml + s*ml_slot, out + s*q_slot. The partials are scratch of
 * `splits` runs per head and slot. The reference cuts every slot's cache into `splits` runs of
 * ceil(stride/splits) rows fixed in cache positions; at head_dim 256 with up to 64 slots this
 * library instead reads the live lengths on the device and deals the batch's 64-key tiles out
 * to one round of CTAs, each slot getting runs in proportion to its live length (still safe to
 * replay from a captured graph: nothing of the plan is baked into the launch). */
int hipml_attn_decode_rows(hipml_stream_t stream, int dtype, const int *pos, const float *q,
                           const void *k_cache, const void *v_cache, float *part_acc,
                           float *part_ml, float *out, int n_heads, int n_kv, int head_dim,
                           int stride, float scale, int splits, int kv_slot_bytes, int acc_slot,
                           int ml_slot, int q_slot, int slots);

/* Launcher::attn_decode_batch (batch_launch.rs:109-209): as above, except that one live slot
 * (slots == 1, live_seq > 0, head_dim 256) partitions over the live length with
 * min(clamp(live_seq/32, 1, 256), splits) splits, as the reference's lone-slot route does. */
int hipml_attn_decode_batch(hipml_stream_t stream, int dtype, const int *pos, const float *q,
                            const void *k_cache, const void *v_cache, float *part_acc,
                            float *part_ml, float *out, int n_heads, int n_kv, int head_dim,
                            int stride, float scale, int splits, int kv_slot_bytes, int acc_slot,
                            int ml_slot, int q_slot, int slots, int live_seq);

/* Bytes of device workspace hipml_attn_chunk needs for a call with these shapes (the staged
 * half-precision image of the visible cache rows). Monotonic in pos0 + tokens. */
size_t hipml_attn_chunk_workspace_bytes(int n_kv, int head_dim, int pos0, int tokens);

/* AttnLayer::chunk_attention_kv (crates/hipml-kernels/src/attn_gpu/imp/attn_chunk_kv.rs:129-305):
 * causal GQA attention of `tokens` query rows at positions pos0..pos0+tokens-1 over cache rows
 * [0, pos0+tokens); row t sees cache rows 0..pos0+t. q and out are f32 [tokens][n_heads*head_dim].
 * kv_dtype: 0 = f32 position-major cache [n_ctx][n_kv*head_dim] (stride unused), 1 = q8_0
 * head-major cache with `stride` rows per KV head, 2 = q4_0 in the same head-major layout.
 * scale is 1/sqrt(head_dim), computed here as the reference does.
 * splits < 2: one pass. splits >= 2: the key axis of every query tile is cut into `splits`
 * slices, partials go to part_acc f32 [splits][qslots][n_heads][head_dim] and part_ml f32
 * [splits][qslots][n_heads][2] with qslots = tokens rounded up to 32, and a combine pass
 * writes out (attn_chunk_split.hip:343-376).
 * mode: 0 = tensor-core kernel with error-compensated half-precision operands (meets the f32
 * tolerance), 1 = tensor-core kernel, single half-precision pass (the reference kernel's own
 * precision), 2 = scalar f32 kernel (any head_dim multiple of 32 up to 256; no workspace),
 * 3 = as 0 but one CTA per query tile instead of CTA pairs (A/B form of the same arithmetic).
 * workspace: device memory of at least hipml_attn_chunk_workspace_bytes(...) for modes 0/1/3,
 * 256-byte aligned. The tensor-core modes want q, out, the caches and part_acc 16-byte aligned
 * and part_ml 8-byte aligned (rows leave the kernel as whole 1 KB bulk copies). */
int hipml_attn_chunk(hipml_stream_t stream, const float *q, const void *k_cache,
                     const void *v_cache, float *out, int n_heads, int n_kv, int head_dim,
                     int pos0, int tokens, int kv_dtype, int stride, float *part_acc,
                     float *part_ml, int splits, int mode, void *workspace,
                     size_t workspace_bytes);

/* The two halves of hipml_attn_chunk's tensor-core modes, for callers that keep the staged
 * image across chunks (no counterpart in the reference, whose kernel converts each K/V tile
 * inside the attention kernel, attn_chunk_wmma.hip:123-154). The workspace is laid out for
 * key_capacity keys per KV head (a multiple of 128; size it with
 * hipml_attn_chunk_workspace_bytes(n_kv, head_dim, 0, key_capacity)) and that capacity must be
 * the same in every call that shares the workspace.
 * hipml_attn_chunk_stage converts cache rows [key_from, key_to) (whole 64-row tiles are
 * rewritten; rows from key_to to the next multiple of 128 are zero-filled).
 * hipml_attn_chunk_staged runs the attention of rows pos0..pos0+tokens-1 over staged rows
 * [0, pos0+tokens); mode 0, 1 or 3 as in hipml_attn_chunk. */
int hipml_attn_chunk_stage(hipml_stream_t stream, const void *k_cache, const void *v_cache,
                           int n_kv, int head_dim, int kv_dtype, int stride, int key_from,
                           int key_to, int key_capacity, void *workspace,
                           size_t workspace_bytes);
int hipml_attn_chunk_staged(hipml_stream_t stream, const float *q, float *out, int n_heads,
                            int n_kv, int head_dim, int pos0, int tokens, float *part_acc,
                            float *part_ml, int splits, int mode, int key_capacity,
                            void *workspace, size_t workspace_bytes);

/* hipml_attn_chunk_staged with the layer's output gate applied where the rows are produced
 * (the attention epilogue, or the combine pass when splits >= 2): out = attention *
 * sigmoid(gate), gate f32 [tokens][n_heads*head_dim]. The reference launches q_gate_f32 over
 * the chunk afterwards (attn_chunk.rs:345-362). */
int hipml_attn_chunk_staged_gated(hipml_stream_t stream, const float *q, float *out,
                                  const float *gate, int n_heads, int n_kv, int head_dim, int pos0,
                                  int tokens, float *part_acc, float *part_ml, int splits, int mode,
                                  int key_capacity, void *workspace, size_t workspace_bytes);

/* Tuning and test knobs of the decode path (no counterpart in the reference).
 * hipml_set_decode_cta_slots: how many CTAs of the tensor-core decode kernel one round of the
 * device holds (default 0 = 2 per SM of the current device); a process that shares the GPU
 * (MPS, a partitioned context) can lower it, and tests use it to reach the plan's limits with
 * small caches. hipml_set_decode_fold_mode: 0 (default) folds inside the split pass, 1 makes
 * the fold a second launch with the same arithmetic (bit-identical output).
 * hipml_decode_plan_quota: host restatement of the multi-slot plan, for tests -- the 64-row
 * tiles per run that the kernel derives from the live lengths `lens[slots]`; the plan's runs,
 * sum over slots of max(1, ceil(ceil(len/64) / quota)) * n_kv, never exceed cta_slots.
 * Returns -1 for arguments outside the plan's domain (cta_slots < 2 * slots * n_kv). */
int hipml_set_decode_cta_slots(int slots);
/* Which body the q8_0 head_dim-256 decode kernel uses where the caller leaves the choice open
 * (selector 0 / 4, and every multi-slot entry): 1 = both contractions on mma.sync (default),
 * 2 = the value contraction on tcgen05.mma kind::i8 with int32 accumulators in TMEM (GQA group
 * <= 6). Selectors 7 and 8 of hipml_attn_decode_kv name the two bodies directly. */
int hipml_set_decode_body(int body);
int hipml_set_decode_fold_mode(int mode);
int hipml_decode_plan_quota(const int *lens, int slots, int splits, int n_kv, int cta_slots);

/* Reads and clears the device status word that kernels with bounded waits set when a wait
 * ran out (0 = none). Synchronises `stream`. Returns HIPML_ERR_DEVICE_STATUS if it was set. */
int hipml_check_device_status(hipml_stream_t stream, int *status);

/* Library build identification: "hipml_cuda <version> sm_100a". */
const char *hipml_version(void);

#ifdef __cplusplus
}
#endif
#endif
