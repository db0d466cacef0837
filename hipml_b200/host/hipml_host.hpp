// C++ mirror of the host-side objects hipml's engine uses on the full-attention path, written
// against the C ABI of include/hipml_cuda.h only. The reference's host is Rust; each type here
// keeps the name, the method names, the argument order and the error sentences of the Rust
// type it stands in for, so a port of the engine reads the same:
//   Buffer        crates/hipml-hip/src/memory.rs:13-120   (f32-counted device buffer)
//   Launcher      crates/hipml-kernels/src/launch.rs:94-229, launch/device/graph_launch.rs:
//                 878-1028, launch/device/batch_launch.rs:22-316
//   launch_kv     crates/hipml-kernels/src/launch_kv.rs:60-280
//   DeepKv        crates/hipml-model/src/gpu/deep_kv.rs:11-162
//   BatchKv       crates/hipml-model/src/gpu/batch/kv.rs:11-118
//   AttnLayer     crates/hipml-kernels/src/attn_gpu/imp/{attn_chunk_kv,attn_cols}.rs and
//                 attn_gpu.rs:885-912 (attention methods only; no weights, no projections)
// Errors follow Rust's Result<(), String>: a Status is empty on success, else the sentence.
#pragma once

#include <cstddef>
#include <cstdint>
#include <string>
#include <vector>

#include "../../include/hipml_cuda.h"

namespace hipml_host {

using Status = std::string;  // "" = Ok(())

// "{what} failed: {code} ({text})", as crates/hipml-hip/src/device.rs:111-124.
Status check(const char *what, int code);

enum class KvDtype { Q8 = 0, Q4 = 1 };
inline int dtype_id(KvDtype d) { return static_cast<int>(d); }
// crates/hipml-core/src/kv.rs:59-90
size_t block_bytes(KvDtype d);
size_t row_bytes(KvDtype d, size_t head_dim);
size_t token_bytes(KvDtype d, size_t n_kv, size_t head_dim, size_t n_layers);
// crates/hipml-core/src/kv.rs:306-329: format-valid filler for bandwidth benches.
std::vector<uint8_t> synthetic_blocks(KvDtype d, size_t n_blocks, uint64_t seed);

// Device buffer counted in f32 elements; frees its allocation when destroyed.
class Buffer {
public:
    Buffer() = default;
    Buffer(const Buffer &) = delete;
    Buffer &operator=(const Buffer &) = delete;
    Buffer(Buffer &&o) noexcept;
    Buffer &operator=(Buffer &&o) noexcept;
    ~Buffer();
    static Status alloc(size_t len, Buffer &out);                       // uninitialised
    static Status from_host(const float *data, size_t len, Buffer &out);
    Status to_host(std::vector<float> &out) const;
    Status upload_bytes(size_t offset, const void *bytes, size_t n) const;
    Status download_bytes(size_t offset, void *bytes, size_t n) const;
    void *as_ptr() const { return ptr_; }
    size_t len() const { return len_; }

private:
    void *ptr_ = nullptr;
    size_t len_ = 0;
};

struct Config {
    size_t n_head = 24, n_head_kv = 4, head_dim = 256;
};

// Stream + the device-resident step buffer [pos, seq, token, 0, p0..p3] (i32 x 8).
class Launcher {
public:
    Launcher() = default;
    ~Launcher();
    static Status create(Launcher &out);
    // launch.rs:144-154: 32-byte asynchronous upload; kernels read step[0] / step[1].
    Status set_step(size_t pos, size_t seq, size_t token);
    const Buffer &step_buf() const { return step_; }
    hipml_stream_t stream() const { return stream_; }
    Status synchronize() const;

    // graph_launch.rs:878-927
    Status kv_encode(size_t dtype, const Buffer &k_in, const Buffer &v_in, const Buffer &k_cache,
                     const Buffer &v_cache, size_t n_kv, size_t head_dim, size_t stride) const;
    Status kv_encode_ptr(size_t dtype, const void *k_ptr, const void *v_ptr, const Buffer &k_cache,
                         const Buffer &v_cache, size_t n_kv, size_t head_dim, size_t stride) const;
    // graph_launch.rs:980-1028
    Status kv_encode_bulk(size_t dtype, const Buffer &k_f32, const Buffer &v_f32,
                          const Buffer &k_cache, const Buffer &v_cache, size_t n_kv,
                          size_t head_dim, size_t stride, size_t start, size_t src0,
                          size_t rows) const;
    // batch_launch.rs:22-49
    Status kv_encode_batch(size_t dtype, const Buffer &k_f32, const Buffer &v_f32,
                           const Buffer &k_cache, const Buffer &v_cache, size_t n_kv,
                           size_t head_dim, size_t stride, const Buffer &pos, size_t slot_bytes,
                           size_t slots) const;
    // batch_launch.rs:109-209
    Status attn_decode_batch(size_t dtype, const Buffer &pos, const Buffer &q,
                             const Buffer &k_cache, const Buffer &v_cache, const Buffer &part_acc,
                             const Buffer &part_ml, const Buffer &out, size_t n_heads, size_t n_kv,
                             size_t head_dim, size_t stride, float scale, size_t splits,
                             size_t kv_slot_bytes, size_t acc_slot, size_t ml_slot, size_t q_slot,
                             size_t slots, size_t live_seq) const;

private:
    hipml_stream_t stream_ = nullptr;
    Buffer step_;
    void *pinned_step_ = nullptr;
};

namespace launch_kv {
// launch_kv.rs:60-129. `seq` is the cache's per-head row stride; the live length is step[1].
Status launch(const Launcher &l, size_t dtype, const Buffer &q, const Buffer &k, const Buffer &v,
              const Buffer &part_acc, const Buffer &part_ml, const Buffer &out, size_t n_heads,
              size_t n_kv, size_t head_dim, size_t seq, float scale, size_t splits, size_t k_off,
              size_t v_off);
Status launch_ptrs(const Launcher &l, size_t dtype, const void *q_ptr, const Buffer &k,
                   const Buffer &v, const Buffer &part_acc, const Buffer &part_ml, void *out_ptr,
                   size_t n_heads, size_t n_kv, size_t head_dim, size_t seq, float scale,
                   size_t splits, size_t k_off, size_t v_off);
// One decode step of a layer: Launcher::kv_encode_ptr_on + launch_ptrs as
// deep_attention makes them (crates/hipml-model/src/gpu/attn_tile.rs:150-224), in one call;
// `gate` may be null. The append position step[0] must be step[1] - 1.
Status step_ptrs(const Launcher &l, size_t dtype, const void *k_row, const void *v_row,
                 const void *q_ptr, const Buffer &k, const Buffer &v, const Buffer &part_acc,
                 const Buffer &part_ml, void *out_ptr, const void *gate, size_t n_heads, size_t n_kv,
                 size_t head_dim, size_t seq, float scale, size_t splits, size_t k_off, size_t v_off);
}  // namespace launch_kv

// One layer's quantised K/V cache plus the split-K scratch (deep_kv.rs:11-99).
class DeepKv {
public:
    static constexpr size_t MAX_SPLITS = 256;
    static Status create(const Config &cfg, size_t seq, KvDtype dtype, DeepKv &out);
    size_t splits(size_t seq) const;          // deep_kv.rs:102-110
    size_t bytes() const;                     // 2 * n_kv * seq * row_bytes
    size_t row_words() const;
    size_t heads() const { return n_kv; }
    Status fill_synthetic(size_t depth, uint64_t seed) const;  // deep_kv.rs:133-144
    KvDtype dtype = KvDtype::Q8;
    size_t seq = 0;
    size_t kernel = 4;
    Buffer k, v, part_acc, part_ml;

private:
    size_t n_kv = 0, head_dim = 0;
};

// Per-layer caches of the batched engine, contiguous across slots (batch/kv.rs:11-118).
size_t attn_splits(size_t stride, size_t slots);  // batch/kv.rs:39-42
class BatchKv {
public:
    static Status create(const Config &cfg, size_t seq, KvDtype dtype, size_t slots, BatchKv &out);
    size_t row() const;
    size_t slot_bytes() const;
    size_t acc_slot() const;
    size_t ml_slot() const;
    size_t bytes() const;
    Status fill_synthetic(const std::vector<size_t> &depths, uint64_t seed) const;
    KvDtype dtype = KvDtype::Q8;
    size_t seq = 0, splits = 0, n_kv = 0, head_dim = 0, slots = 0;
    Buffer k, v, part_acc, part_ml;
};

// Quantised-KV decode of `cols` consecutive columns of one sequence (speculative verify):
// one launch per group of columns with the same split count, every column bit-identical to
// its one-column launch (crates/hipml-model/src/gpu/attn_tile.rs:225-295). pos_buf holds
// (position, length) pairs per column; scratch slices are acc_slot / ml_slot floats apart.
Status deep_attention_cols(const Launcher &l, const Config &cfg, const DeepKv &dk, size_t pos0,
                           size_t cols, const void *q_ptr, void *out_ptr, const Buffer &pos_buf,
                           void *part_acc, void *part_ml, size_t acc_slot, size_t ml_slot,
                           bool &handled);

// The attention half of a prefix snapshot (crates/hipml-model/src/gpu/prefix.rs:30-43): the
// live rows [0, rows) of every KV head, between caches of `src_seq` and `dst_seq` rows per head.
Status kv_prefix_copy(const Launcher &l, const Buffer &dst, const Buffer &src, size_t n_kv,
                      size_t row_bytes, size_t dst_seq, size_t src_seq, size_t rows);

// Front end and tail of the attention layer on explicit row pointers (a row block holds
// several slots' tails; crates/hipml-kernels/src/attn_gpu/imp/attn_rows.rs:21-203).
struct FrontDims {
    size_t n_head = 24, n_kv = 4, head_dim = 256, n_rot = 64;
    int sections[4] = {11, 11, 10, 0};
    float rope_base = 1e7f, eps = 1e-6f;
};
// attn_rows.rs:21-95: q|gate split, per-head RMS norm and M-RoPE of `tokens` rows at pos0.
Status chunk_front_rows(const Launcher &l, const FrontDims &d, const void *qg, void *k, void *q,
                        void *gate, const Buffer &q_norm, const Buffer &k_norm, size_t pos0,
                        size_t tokens);
// attn_rows.rs:97-148: quantise-append of the block's rows into one slot's cache.
Status kv_encode_bulk_rows(const Launcher &l, const void *k, const void *v, void *k_cache,
                           void *v_cache, size_t dtype, size_t n_kv, size_t head_dim, size_t seq,
                           size_t start, size_t rows);
// The two above in one pass (no counterpart in the reference).
Status chunk_front_append_rows(const Launcher &l, const FrontDims &d, const void *qg, const void *k,
                               const void *v, void *q, void *gate, const Buffer &q_norm,
                               const Buffer &k_norm, void *k_cache, void *v_cache, size_t seq,
                               size_t pos0, size_t tokens);
// attn_chunk.rs:345-362: out *= sigmoid(gate) over `tokens` rows.
Status q_gate_rows(const Launcher &l, const FrontDims &d, void *out, const void *gate, size_t tokens);

// Prefill split policy (crates/hipml-model/src/gpu/attn_tile.rs:138-151).
size_t split_count(size_t configured, size_t pos0, size_t split_min = 8192);

struct AttnDims {
    size_t n_head = 24, n_kv = 4, head_dim = 256, width = 1024, n_ctx = 0;
};

// The attention methods of the reference's per-layer object. It owns the f32 cache pair
// (kv_k, kv_v: [n_ctx][width]) and the workspace the tensor-core chunk kernel stages into.
class AttnLayer {
public:
    static Status create(const Config &cfg, size_t n_ctx, AttnLayer &out);
    bool q8_chunk_supported() const;  // attn_chunk_kv.rs:35-38
    // attn_chunk_kv.rs:112-123, 44-62, 72-107
    Status chunk_attention(const Launcher &l, const Buffer &q, const Buffer &kc, const Buffer &vc,
                           const Buffer &out, size_t pos0, size_t tokens) const;
    Status chunk_attention_q8(const Launcher &l, const Buffer &q, const Buffer &kc,
                              const Buffer &vc, const Buffer &out, size_t pos0, size_t tokens,
                              size_t dtype, size_t stride) const;
    Status chunk_attention_q8_split(const Launcher &l, const Buffer &q, const Buffer &kc,
                                    const Buffer &vc, const Buffer &out, size_t pos0,
                                    size_t tokens, size_t dtype, size_t stride,
                                    const Buffer &part_acc, const Buffer &part_ml,
                                    size_t splits) const;
    // attn_gpu.rs:885-912: copy one K/V row into the f32 caches at step[0].
    Status append_at(const Launcher &l, const void *k_ptr, const void *v_ptr) const;
    // attn_cols.rs:15-31, 34-64, 66-173
    void split_geom(size_t &splits, size_t &per) const;
    void split_scratch(size_t rows, size_t &acc, size_t &ml) const;
    Status append_rows(const Launcher &l, const Buffer &k, const Buffer &v, size_t rows,
                       size_t pos0) const;
    Status attention_cols(const Launcher &l, const void *q, void *out, const Buffer &part_acc,
                          const Buffer &part_ml, size_t pos0, size_t rows) const;
    // 0 compensated (default), 1 single-pass f16, 2 scalar f32 (the reference's HIPML_ATTN_F32 A/B).
    int mode = 0;
    AttnDims dims;
    Buffer kv_k, kv_v;

private:
    Status chunk_attention_kv(const Launcher &l, const Buffer &q, const Buffer &kc,
                              const Buffer &vc, const Buffer &out, size_t pos0, size_t tokens,
                              size_t dtype, size_t stride, const Buffer *part_acc,
                              const Buffer *part_ml, size_t splits) const;
    Buffer workspace_;
    size_t workspace_bytes_ = 0;
};

}  // namespace hipml_host
