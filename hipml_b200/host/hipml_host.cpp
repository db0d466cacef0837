// Implementation of the host-side mirror (see hipml_host.hpp). Uses only the C ABI.
#include "hipml_host.hpp"

#include <algorithm>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstring>

namespace hipml_host {

Status check(const char *what, int code) {
    if (code == 0) return {};
    const char *text =
        code >= HIPML_ERR_BASE ? hipml_last_error_message() : hipml_get_error_string(code);
    if (code >= HIPML_ERR_BASE) return std::string(text);  // the launcher's own sentence
    char buf[640];
    snprintf(buf, sizeof(buf), "%s failed: %d (%s)", what, code, text ? text : "");
    return buf;
}

static Status fmt(const char *f, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, f);
    vsnprintf(buf, sizeof(buf), f, ap);
    va_end(ap);
    return buf;
}

// ---- format helpers (crates/hipml-core/src/kv.rs) ---------------------------------------

size_t block_bytes(KvDtype d) { return d == KvDtype::Q8 ? 34 : 18; }

size_t row_bytes(KvDtype d, size_t head_dim) { return head_dim / 32 * block_bytes(d); }

size_t token_bytes(KvDtype d, size_t n_kv, size_t head_dim, size_t n_layers) {
    return 2 * n_kv * n_layers * row_bytes(d, head_dim);
}

// f32 -> f16 bits, round to nearest even; only used on the filler's scales (normal range).
static uint16_t f32_to_f16_bits(float v) {
    uint32_t x;
    memcpy(&x, &v, 4);
    const uint16_t sign = (uint16_t)((x >> 16) & 0x8000u);
    int e = (int)((x >> 23) & 0xff) - 112;
    uint32_t mant = x & 0x007fffffu;
    if (e >= 0x1f) return (uint16_t)(sign | 0x7c00u);
    if (e <= 0) {
        if (e < -10) return sign;
        mant |= 0x00800000u;
        const int shift = 14 - e;
        uint32_t m = mant >> shift;
        const uint32_t rem = mant & ((1u << shift) - 1u), half = 1u << (shift - 1);
        if (rem > half || (rem == half && (m & 1u))) m++;
        return (uint16_t)(sign | m);
    }
    uint32_t m = mant >> 13;
    const uint32_t rem = mant & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (m & 1u))) {
        if (++m == 0x400u) {
            m = 0;
            if (++e >= 0x1f) return (uint16_t)(sign | 0x7c00u);
        }
    }
    return (uint16_t)(sign | ((uint32_t)e << 10) | m);
}

static uint64_t xorshift64star(uint64_t &s) {
    s ^= s >> 12;
    s ^= s << 25;
    s ^= s >> 27;
    return s * 0x2545F4914F6CDD1DULL;
}

std::vector<uint8_t> synthetic_blocks(KvDtype d, size_t n_blocks, uint64_t seed) {
    const size_t bb = block_bytes(d);
    std::vector<uint8_t> out(n_blocks * bb);
    uint64_t s = seed | 1;
    for (size_t b = 0; b < n_blocks; b++) {
        uint8_t *blk = out.data() + b * bb;
        // scale in [0.01, 0.05): a normal f16, so the hot loop sees no denormals
        const float scale = 0.01f + (float)(xorshift64star(s) % 1000) * 0.00004f;
        const uint16_t h = f32_to_f16_bits(scale);
        blk[0] = (uint8_t)(h & 0xff);
        blk[1] = (uint8_t)(h >> 8);
        for (size_t j = 0; j + 2 < bb; j++) blk[2 + j] = (uint8_t)(xorshift64star(s) >> 24);
    }
    return out;
}

// ---- Buffer -----------------------------------------------------------------------------

Buffer::Buffer(Buffer &&o) noexcept : ptr_(o.ptr_), len_(o.len_) {
    o.ptr_ = nullptr;
    o.len_ = 0;
}

Buffer &Buffer::operator=(Buffer &&o) noexcept {
    if (this != &o) {
        if (ptr_) hipml_free(ptr_);
        ptr_ = o.ptr_;
        len_ = o.len_;
        o.ptr_ = nullptr;
        o.len_ = 0;
    }
    return *this;
}

Buffer::~Buffer() {
    if (ptr_) hipml_free(ptr_);
}

Status Buffer::alloc(size_t len, Buffer &out) {
    void *p = nullptr;
    if (Status s = check("hipMalloc", hipml_malloc(&p, std::max<size_t>(len, 1) * 4)); !s.empty())
        return s;
    out = Buffer();
    out.ptr_ = p;
    out.len_ = len;
    return {};
}

Status Buffer::from_host(const float *data, size_t len, Buffer &out) {
    if (Status s = alloc(len, out); !s.empty()) return s;
    return check("hipMemcpy", hipml_memcpy(out.ptr_, data, len * 4, HIPML_MEMCPY_HOST_TO_DEVICE));
}

Status Buffer::to_host(std::vector<float> &out) const {
    out.resize(len_);
    return check("hipMemcpy", hipml_memcpy(out.data(), ptr_, len_ * 4, HIPML_MEMCPY_DEVICE_TO_HOST));
}

Status Buffer::upload_bytes(size_t offset, const void *bytes, size_t n) const {
    if (offset + n > len_ * 4)
        return fmt("upload of %zu bytes at %zu beyond buffer %zu", n, offset, len_ * 4);
    return check("hipMemcpy", hipml_memcpy((char *)ptr_ + offset, bytes, n, HIPML_MEMCPY_HOST_TO_DEVICE));
}

Status Buffer::download_bytes(size_t offset, void *bytes, size_t n) const {
    if (offset + n > len_ * 4)
        return fmt("download of %zu bytes at %zu beyond buffer %zu", n, offset, len_ * 4);
    return check("hipMemcpy", hipml_memcpy(bytes, (const char *)ptr_ + offset, n, HIPML_MEMCPY_DEVICE_TO_HOST));
}

// ---- Launcher ---------------------------------------------------------------------------

Launcher::~Launcher() {
    if (pinned_step_) hipml_host_free(pinned_step_);
    if (stream_) hipml_stream_destroy(stream_);
}

Status Launcher::create(Launcher &out) {
    if (Status s = check("hipInit", hipml_init(0)); !s.empty()) return s;
    if (Status s = check("hipStreamCreate", hipml_stream_create(&out.stream_)); !s.empty()) return s;
    if (Status s = Buffer::alloc(8, out.step_); !s.empty()) return s;
    if (Status s = check("hipHostMalloc", hipml_host_alloc(&out.pinned_step_, 32)); !s.empty()) return s;
    return out.set_step(0, 1, 0);
}

Status Launcher::set_step(size_t pos, size_t seq, size_t token) {
    // The previous upload must have left the pinned staging words before they are rewritten.
    if (Status s = check("hipStreamSynchronize", hipml_stream_synchronize(stream_)); !s.empty()) return s;
    int32_t *w = static_cast<int32_t *>(pinned_step_);
    const int32_t p = (int32_t)pos;
    const int32_t words[8] = {p, (int32_t)seq, (int32_t)token, 0, p, p, p, p};
    memcpy(w, words, 32);
    return check("hipMemcpyAsync", hipml_memcpy_async(step_.as_ptr(), w, 32, HIPML_MEMCPY_HOST_TO_DEVICE, stream_));
}

Status Launcher::synchronize() const {
    return check("hipStreamSynchronize", hipml_stream_synchronize(stream_));
}

Status Launcher::kv_encode(size_t dtype, const Buffer &k_in, const Buffer &v_in, const Buffer &k_cache,
                           const Buffer &v_cache, size_t n_kv, size_t head_dim, size_t stride) const {
    return kv_encode_ptr(dtype, k_in.as_ptr(), v_in.as_ptr(), k_cache, v_cache, n_kv, head_dim, stride);
}

Status Launcher::kv_encode_ptr(size_t dtype, const void *k_ptr, const void *v_ptr, const Buffer &k_cache,
                               const Buffer &v_cache, size_t n_kv, size_t head_dim, size_t stride) const {
    return check("kv_encode",
                 hipml_kv_encode(stream_, (const int *)step_.as_ptr(), (int)dtype, (const float *)k_ptr,
                                 (const float *)v_ptr, k_cache.as_ptr(), v_cache.as_ptr(), (int)n_kv,
                                 (int)head_dim, (int)stride));
}

Status Launcher::kv_encode_bulk(size_t dtype, const Buffer &k_f32, const Buffer &v_f32, const Buffer &k_cache,
                                const Buffer &v_cache, size_t n_kv, size_t head_dim, size_t stride,
                                size_t start, size_t src0, size_t rows) const {
    return check("kv_encode_bulk",
                 hipml_kv_encode_bulk(stream_, (int)dtype, (const float *)k_f32.as_ptr(),
                                      (const float *)v_f32.as_ptr(), k_cache.as_ptr(), v_cache.as_ptr(),
                                      (int)n_kv, (int)head_dim, (int)stride, (int)start, (int)src0, (int)rows));
}

Status Launcher::kv_encode_batch(size_t dtype, const Buffer &k_f32, const Buffer &v_f32, const Buffer &k_cache,
                                 const Buffer &v_cache, size_t n_kv, size_t head_dim, size_t stride,
                                 const Buffer &pos, size_t slot_bytes, size_t slots) const {
    return check("kv_encode_batch",
                 hipml_kv_encode_rows(stream_, (int)dtype, (const float *)k_f32.as_ptr(),
                                      (const float *)v_f32.as_ptr(), k_cache.as_ptr(), v_cache.as_ptr(),
                                      (int)n_kv, (int)head_dim, (int)stride, (const int *)pos.as_ptr(),
                                      (int)slot_bytes, (int)slots));
}

Status Launcher::attn_decode_batch(size_t dtype, const Buffer &pos, const Buffer &q, const Buffer &k_cache,
                                   const Buffer &v_cache, const Buffer &part_acc, const Buffer &part_ml,
                                   const Buffer &out, size_t n_heads, size_t n_kv, size_t head_dim,
                                   size_t stride, float scale, size_t splits, size_t kv_slot_bytes,
                                   size_t acc_slot, size_t ml_slot, size_t q_slot, size_t slots,
                                   size_t live_seq) const {
    return check("attn_decode_batch",
                 hipml_attn_decode_batch(stream_, (int)dtype, (const int *)pos.as_ptr(), (const float *)q.as_ptr(),
                                         k_cache.as_ptr(), v_cache.as_ptr(), (float *)part_acc.as_ptr(),
                                         (float *)part_ml.as_ptr(), (float *)out.as_ptr(), (int)n_heads,
                                         (int)n_kv, (int)head_dim, (int)stride, scale, (int)splits,
                                         (int)kv_slot_bytes, (int)acc_slot, (int)ml_slot, (int)q_slot,
                                         (int)slots, (int)live_seq));
}

// ---- launch_kv --------------------------------------------------------------------------

namespace launch_kv {

Status launch(const Launcher &l, size_t dtype, const Buffer &q, const Buffer &k, const Buffer &v,
              const Buffer &part_acc, const Buffer &part_ml, const Buffer &out, size_t n_heads,
              size_t n_kv, size_t head_dim, size_t seq, float scale, size_t splits, size_t k_off,
              size_t v_off) {
    return launch_ptrs(l, dtype, q.as_ptr(), k, v, part_acc, part_ml, out.as_ptr(), n_heads, n_kv,
                       head_dim, seq, scale, splits, k_off, v_off);
}

Status launch_ptrs(const Launcher &l, size_t dtype, const void *q_ptr, const Buffer &k,
                   const Buffer &v, const Buffer &part_acc, const Buffer &part_ml, void *out_ptr,
                   size_t n_heads, size_t n_kv, size_t head_dim, size_t seq, float scale,
                   size_t splits, size_t k_off, size_t v_off) {
    return check("attn_decode_kv",
                 hipml_attn_decode_kv(l.stream(), (const int *)l.step_buf().as_ptr(), (int)dtype,
                                      (const float *)q_ptr, k.as_ptr(), v.as_ptr(),
                                      (float *)part_acc.as_ptr(), (float *)part_ml.as_ptr(),
                                      (float *)out_ptr, (int)n_heads, (int)n_kv, (int)head_dim,
                                      (int)seq, scale, (int)std::max<size_t>(splits, 1), k_off, v_off));
}

Status step_ptrs(const Launcher &l, size_t dtype, const void *k_row, const void *v_row,
                 const void *q_ptr, const Buffer &k, const Buffer &v, const Buffer &part_acc,
                 const Buffer &part_ml, void *out_ptr, const void *gate, size_t n_heads, size_t n_kv,
                 size_t head_dim, size_t seq, float scale, size_t splits, size_t k_off, size_t v_off) {
    return check("attn_decode_kv_append",
                 hipml_attn_decode_kv_append(l.stream(), (const int *)l.step_buf().as_ptr(), (int)dtype,
                                             (const float *)k_row, (const float *)v_row,
                                             (const float *)q_ptr, k.as_ptr(), v.as_ptr(),
                                             (float *)part_acc.as_ptr(), (float *)part_ml.as_ptr(),
                                             (float *)out_ptr, (const float *)gate, (int)n_heads,
                                             (int)n_kv, (int)head_dim, (int)seq, scale,
                                             (int)std::max<size_t>(splits, 1), k_off, v_off));
}

}  // namespace launch_kv

// ---- DeepKv -----------------------------------------------------------------------------

static size_t clampz(size_t v, size_t lo, size_t hi) { return std::min(std::max(v, lo), hi); }

Status DeepKv::create(const Config &cfg, size_t seq, KvDtype dtype, DeepKv &out) {
    const size_t row = row_bytes(dtype, cfg.head_dim);
    const size_t f32s = (cfg.n_head_kv * seq * row + 3) / 4;
    const size_t group = cfg.n_head / cfg.n_head_kv;
    out.dtype = dtype;
    out.seq = seq;
    // deep_kv.rs:62-71: the whole-group kernel family at head_dim 256 and a group of at most 8
    out.kernel = (dtype == KvDtype::Q8 && cfg.head_dim == 256 && group <= 8)
                     ? (group >= 7 ? 7 : 4)
                     : (size_t)dtype_id(dtype);
    out.n_kv = cfg.n_head_kv;
    out.head_dim = cfg.head_dim;
    if (Status s = Buffer::alloc(f32s, out.k); !s.empty()) return s;
    if (Status s = Buffer::alloc(f32s, out.v); !s.empty()) return s;
    if (Status s = Buffer::alloc(cfg.n_head * MAX_SPLITS * cfg.head_dim, out.part_acc); !s.empty()) return s;
    return Buffer::alloc(cfg.n_head * MAX_SPLITS * 2, out.part_ml);
}

size_t DeepKv::splits(size_t seq_now) const {
    if (kernel >= 4) return std::max(clampz(seq_now / 8, 1, 128), clampz(seq_now / 64, 1, 256));
    return clampz(seq_now / 64, 1, 64);
}

size_t DeepKv::bytes() const { return 2 * n_kv * seq * row_bytes(dtype, head_dim); }

size_t DeepKv::row_words() const { return row_bytes(dtype, head_dim) / 4; }

Status DeepKv::fill_synthetic(size_t depth, uint64_t seed) const {
    const std::vector<uint8_t> pattern = synthetic_blocks(dtype, depth * (head_dim / 32), seed);
    const size_t row = row_bytes(dtype, head_dim);
    for (size_t h = 0; h < n_kv; h++) {
        const size_t off = h * seq * row;
        if (Status s = k.upload_bytes(off, pattern.data(), pattern.size()); !s.empty()) return s;
        if (Status s = v.upload_bytes(off, pattern.data(), pattern.size()); !s.empty()) return s;
    }
    return {};
}

// ---- BatchKv ----------------------------------------------------------------------------

size_t attn_splits(size_t stride, size_t slots) {
    const size_t per = 64 * std::max<size_t>((slots + 3) / 4, 1);
    return clampz((stride + per - 1) / per, 1, 256);
}

Status BatchKv::create(const Config &cfg, size_t seq, KvDtype dtype, size_t slots, BatchKv &out) {
    if (slots == 0 || slots > 32) return fmt("slots %zu: the batched engine runs 1..=32 slots", slots);
    out.dtype = dtype;
    out.seq = seq;
    out.splits = attn_splits(seq, slots);
    out.n_kv = cfg.n_head_kv;
    out.head_dim = cfg.head_dim;
    out.slots = slots;
    const size_t cache_f32 = (slots * out.slot_bytes() + 3) / 4;
    if (Status s = Buffer::alloc(cache_f32, out.k); !s.empty()) return s;
    if (Status s = Buffer::alloc(cache_f32, out.v); !s.empty()) return s;
    if (Status s = Buffer::alloc(slots * cfg.n_head * out.splits * cfg.head_dim, out.part_acc); !s.empty())
        return s;
    return Buffer::alloc(slots * cfg.n_head * out.splits * 2, out.part_ml);
}

size_t BatchKv::row() const { return row_bytes(dtype, head_dim); }
size_t BatchKv::slot_bytes() const { return n_kv * seq * row(); }
size_t BatchKv::acc_slot() const { return part_acc.len() / slots; }
size_t BatchKv::ml_slot() const { return part_ml.len() / slots; }
size_t BatchKv::bytes() const { return 2 * slots * slot_bytes(); }

Status BatchKv::fill_synthetic(const std::vector<size_t> &depths, uint64_t seed) const {
    for (size_t b = 0; b < depths.size(); b++) {
        const std::vector<uint8_t> pattern = synthetic_blocks(dtype, depths[b] * (head_dim / 32), seed);
        seed = seed * 6364136223846793005ULL + 1;
        for (size_t h = 0; h < n_kv; h++) {
            const size_t off = b * slot_bytes() + h * seq * row();
            if (Status s = k.upload_bytes(off, pattern.data(), pattern.size()); !s.empty()) return s;
            if (Status s = v.upload_bytes(off, pattern.data(), pattern.size()); !s.empty()) return s;
        }
    }
    return {};
}

size_t split_count(size_t configured, size_t pos0, size_t split_min) {
    return (configured >= 2 && pos0 >= split_min) ? configured : 1;
}

// ---- AttnLayer --------------------------------------------------------------------------

Status AttnLayer::create(const Config &cfg, size_t n_ctx, AttnLayer &out) {
    out.dims.n_head = cfg.n_head;
    out.dims.n_kv = cfg.n_head_kv;
    out.dims.head_dim = cfg.head_dim;
    out.dims.width = cfg.n_head_kv * cfg.head_dim;
    out.dims.n_ctx = n_ctx;
    if (Status s = Buffer::alloc(n_ctx * out.dims.width, out.kv_k); !s.empty()) return s;
    if (Status s = Buffer::alloc(n_ctx * out.dims.width, out.kv_v); !s.empty()) return s;
    out.workspace_bytes_ =
        hipml_attn_chunk_workspace_bytes((int)cfg.n_head_kv, (int)cfg.head_dim, 0, (int)n_ctx);
    if (out.workspace_bytes_ == 0) return {};  // shapes only the scalar kernel serves
    return Buffer::alloc((out.workspace_bytes_ + 3) / 4, out.workspace_);
}

bool AttnLayer::q8_chunk_supported() const {
    return dims.head_dim == 256 && dims.n_kv > 0 && dims.n_head % dims.n_kv == 0 &&
           dims.n_head / dims.n_kv <= 8;
}

Status AttnLayer::chunk_attention(const Launcher &l, const Buffer &q, const Buffer &kc, const Buffer &vc,
                                  const Buffer &out, size_t pos0, size_t tokens) const {
    return chunk_attention_kv(l, q, kc, vc, out, pos0, tokens, 0, 0, nullptr, nullptr, 1);
}

Status AttnLayer::chunk_attention_q8(const Launcher &l, const Buffer &q, const Buffer &kc, const Buffer &vc,
                                     const Buffer &out, size_t pos0, size_t tokens, size_t dtype,
                                     size_t stride) const {
    if (!q8_chunk_supported() || dtype < 1 || dtype > 2)
        return "quantized chunk attention: only head_dim 256 with a q8/q4 cache";
    return chunk_attention_kv(l, q, kc, vc, out, pos0, tokens, dtype, stride, nullptr, nullptr, 1);
}

Status AttnLayer::chunk_attention_q8_split(const Launcher &l, const Buffer &q, const Buffer &kc,
                                           const Buffer &vc, const Buffer &out, size_t pos0, size_t tokens,
                                           size_t dtype, size_t stride, const Buffer &part_acc,
                                           const Buffer &part_ml, size_t splits) const {
    if (!q8_chunk_supported() || dtype < 1 || dtype > 2)
        return "quantized chunk attention: only head_dim 256 with a q8/q4 cache";
    if (splits < 2) return chunk_attention_kv(l, q, kc, vc, out, pos0, tokens, dtype, stride, nullptr, nullptr, 1);
    return chunk_attention_kv(l, q, kc, vc, out, pos0, tokens, dtype, stride, &part_acc, &part_ml, splits);
}

Status AttnLayer::chunk_attention_kv(const Launcher &l, const Buffer &q, const Buffer &kc, const Buffer &vc,
                                     const Buffer &out, size_t pos0, size_t tokens, size_t dtype,
                                     size_t stride, const Buffer *part_acc, const Buffer *part_ml,
                                     size_t splits) const {
    const int use_mode = (dims.head_dim == 256 && workspace_bytes_ > 0) ? mode : 2;
    return check("chunk_attention",
                 hipml_attn_chunk(l.stream(), (const float *)q.as_ptr(), kc.as_ptr(), vc.as_ptr(),
                                  (float *)out.as_ptr(), (int)dims.n_head, (int)dims.n_kv, (int)dims.head_dim,
                                  (int)pos0, (int)tokens, (int)dtype, (int)stride,
                                  part_acc ? (float *)part_acc->as_ptr() : nullptr,
                                  part_ml ? (float *)part_ml->as_ptr() : nullptr, (int)splits, use_mode,
                                  workspace_.as_ptr(), workspace_bytes_));
}

Status AttnLayer::append_at(const Launcher &l, const void *k_ptr, const void *v_ptr) const {
    return check("kv_append_f32",
                 hipml_kv_append_f32(l.stream(), (const int *)l.step_buf().as_ptr(), (float *)kv_k.as_ptr(),
                                     (float *)kv_v.as_ptr(), (const float *)k_ptr, (const float *)v_ptr,
                                     (int)dims.width));
}

void AttnLayer::split_geom(size_t &splits, size_t &per) const {
    splits = clampz((dims.n_ctx + 31) / 32, 1, 64);
    per = (dims.n_ctx + splits - 1) / splits;
}

void AttnLayer::split_scratch(size_t rows, size_t &acc, size_t &ml) const {
    size_t splits, per;
    split_geom(splits, per);
    acc = rows * dims.n_head * splits * dims.head_dim;
    ml = rows * dims.n_head * splits * 2;
}

Status AttnLayer::append_rows(const Launcher &l, const Buffer &k, const Buffer &v, size_t rows,
                              size_t pos0) const {
    return check("kv_append_cols_f32",
                 hipml_kv_append_cols_f32(l.stream(), (float *)kv_k.as_ptr(), (float *)kv_v.as_ptr(),
                                          (const float *)k.as_ptr(), (const float *)v.as_ptr(), (int)pos0,
                                          (int)rows, (int)dims.width));
}

Status AttnLayer::attention_cols(const Launcher &l, const void *q, void *out, const Buffer &part_acc,
                                 const Buffer &part_ml, size_t pos0, size_t rows) const {
    size_t need_acc, need_ml;
    split_scratch(rows, need_acc, need_ml);
    if (part_acc.len() < need_acc || part_ml.len() < need_ml)
        return fmt("attention scratch: %zu / %zu values for %zu columns", part_acc.len(), part_ml.len(), rows);
    return check("attention_cols",
                 hipml_attn_decode_cols_f32(l.stream(), (const float *)q, (const float *)kv_k.as_ptr(),
                                            (const float *)kv_v.as_ptr(), (float *)part_acc.as_ptr(),
                                            (float *)part_ml.as_ptr(), (float *)out, (int)dims.n_head,
                                            (int)dims.n_kv, (int)dims.head_dim, (int)dims.n_ctx, (int)pos0,
                                            (int)rows));
}

Status deep_attention_cols(const Launcher &l, const Config &cfg, const DeepKv &dk, size_t pos0,
                           size_t cols, const void *q_ptr, void *out_ptr, const Buffer &pos_buf,
                           void *part_acc, void *part_ml, size_t acc_slot, size_t ml_slot,
                           bool &handled) {
    handled = false;
    if (dk.kernel != 4 && dk.kernel != 0) return {};   // only the warp entry has a batched form
    if (dk.dtype != KvDtype::Q8) return {};
    const size_t qw = cfg.n_head * cfg.head_dim;
    const float scale = 1.0f / std::sqrt((float)cfg.head_dim);
    size_t c0 = 0;
    while (c0 < cols) {
        // columns that share a split count go out together, so that each column's arithmetic
        // is the one-column launch's
        const size_t splits = dk.splits(pos0 + c0 + 1);
        size_t c1 = c0 + 1;
        while (c1 < cols && dk.splits(pos0 + c1 + 1) == splits) c1++;
        Status s = check("attn_decode_cols",
                         hipml_attn_decode_cols(l.stream(), 0, (const int *)pos_buf.as_ptr() + 2 * c0,
                                                (const float *)q_ptr + c0 * qw, dk.k.as_ptr(),
                                                dk.v.as_ptr(), (float *)part_acc + c0 * acc_slot,
                                                (float *)part_ml + c0 * ml_slot,
                                                (float *)out_ptr + c0 * qw, (int)cfg.n_head,
                                                (int)cfg.n_head_kv, (int)cfg.head_dim, (int)dk.seq, scale,
                                                (int)splits, (int)(c1 - c0), (int)acc_slot, (int)ml_slot,
                                                (int)qw));
        if (!s.empty()) return s;
        c0 = c1;
    }
    handled = true;
    return {};
}

Status kv_prefix_copy(const Launcher &l, const Buffer &dst, const Buffer &src, size_t n_kv,
                      size_t row_bytes, size_t dst_seq, size_t src_seq, size_t rows) {
    return check("kv_rows_copy", hipml_kv_rows_copy(l.stream(), dst.as_ptr(), src.as_ptr(), (int)n_kv,
                                                    (int)row_bytes, (int)dst_seq, (int)src_seq,
                                                    (int)rows));
}

Status chunk_front_rows(const Launcher &l, const FrontDims &d, const void *qg, void *k, void *q,
                        void *gate, const Buffer &q_norm, const Buffer &k_norm, size_t pos0,
                        size_t tokens) {
    if (d.head_dim > 256) return std::string("row attention: unsupported head dimension");
    Status s = check("qg_split_chunk",
                     hipml_qg_split_chunk(l.stream(), (const float *)qg, (float *)q, (float *)gate,
                                          (int)d.n_head, (int)d.head_dim, (int)tokens));
    if (!s.empty()) return s;
    return check("norm_rope_chunk",
                 hipml_norm_rope_chunk(l.stream(), (float *)q, (float *)k, (const float *)q_norm.as_ptr(),
                                       (const float *)k_norm.as_ptr(), (int)d.n_head, (int)d.n_kv,
                                       (int)d.head_dim, (int)d.n_rot, d.rope_base, d.eps, (int)pos0,
                                       (int)tokens));
}

Status kv_encode_bulk_rows(const Launcher &l, const void *k, const void *v, void *k_cache,
                           void *v_cache, size_t dtype, size_t n_kv, size_t head_dim, size_t seq,
                           size_t start, size_t rows) {
    return check("kv_encode_bulk",
                 hipml_kv_encode_bulk(l.stream(), (int)dtype, (const float *)k, (const float *)v, k_cache,
                                      v_cache, (int)n_kv, (int)head_dim, (int)seq, (int)start, 0,
                                      (int)rows));
}

Status chunk_front_append_rows(const Launcher &l, const FrontDims &d, const void *qg, const void *k,
                               const void *v, void *q, void *gate, const Buffer &q_norm,
                               const Buffer &k_norm, void *k_cache, void *v_cache, size_t seq,
                               size_t pos0, size_t tokens) {
    return check("attn_front_append_q8",
                 hipml_attn_front_append_q8(l.stream(), (const float *)qg, (const float *)k,
                                            (const float *)v, (float *)q, (float *)gate, nullptr,
                                            (const float *)q_norm.as_ptr(),
                                            (const float *)k_norm.as_ptr(), k_cache, v_cache,
                                            (int)d.n_head, (int)d.n_kv, (int)d.head_dim, (int)d.n_rot,
                                            nullptr, nullptr, nullptr, (int)pos0, (int)tokens, (int)seq,
                                            d.rope_base, d.eps));
}

Status q_gate_rows(const Launcher &l, const FrontDims &d, void *out, const void *gate, size_t tokens) {
    return check("q_gate", hipml_q_gate(l.stream(), (const float *)out, (const float *)gate, (float *)out,
                                        (long long)(d.n_head * d.head_dim * tokens)));
}

}  // namespace hipml_host
