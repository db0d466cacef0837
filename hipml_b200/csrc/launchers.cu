// Section B of the C ABI: the attention launchers. Each function validates its
// arguments with the reference launcher's own rules and messages, then launches on the
// caller's stream. Reference launch code: crates/hipml-kernels/src/launch_kv.rs:110-280,
// crates/hipml-kernels/src/launch/device/graph_launch.rs:878-1028,
// crates/hipml-kernels/src/launch/device/batch_launch.rs:22-316,
// crates/hipml-kernels/src/attn_gpu/imp/attn_chunk_kv.rs:129-305.
#include <atomic>

#include "params.cuh"

using namespace hipml;

namespace {

constexpr float kLog2e = 1.4426950408889634f;

int check_encode(int dtype, int n_kv, int head_dim, int stride) {
    if (dtype != 0 && dtype != 1)
        return fail(HIPML_ERR_INVALID_ARGUMENT, "unknown KV dtype %d", dtype);
    if (n_kv <= 0 || stride <= 0)
        return fail(HIPML_ERR_INVALID_ARGUMENT, "n_kv %d / stride %d must be positive", n_kv, stride);
    if (head_dim % 32 != 0 || head_dim < 32 || head_dim > 256)
        return fail(HIPML_ERR_INVALID_ARGUMENT, "head_dim %d: must be 32..=256, multiple of 32",
                    head_dim);
    return 0;
}

// Live runs per KV head of the single-stream split pass: one round of the device's CTA slots
// (two CTAs per SM), so that every CTA streams one long run instead of several short ones.
// Cached per device; hipml_set_decode_cta_slots overrides it for every device.
std::atomic<int> g_cta_slots_override{0};
int decode_cta_slots() {
    const int forced = g_cta_slots_override.load();
    if (forced > 0) return forced;
    static std::atomic<int> cached[64];
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    int slots = cached[dev].load();
    if (slots == 0) {
        int sms = 0;
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
            sms = 148;
        slots = 2 * sms;
        cached[dev].store(slots);
    }
    return slots;
}
int decode_run_cap(int n_kv) {
    const int cap = decode_cta_slots() / (n_kv > 0 ? n_kv : 1);
    return cap < 1 ? 1 : cap;
}

int check_heads(int n_heads, int n_kv, int head_dim) {
    if (n_kv <= 0 || n_heads % n_kv != 0)
        return fail(HIPML_ERR_INVALID_ARGUMENT, "n_heads %d is not a multiple of n_kv %d", n_heads,
                    n_kv);
    const int group = n_heads / n_kv;
    if (group > 8)
        return fail(HIPML_ERR_INVALID_ARGUMENT, "GQA group %d > 8: one block holds at most 8 warps",
                    group);
    if (head_dim % 32 != 0 || head_dim < 32 || head_dim > 256)
        return fail(HIPML_ERR_INVALID_ARGUMENT, "head_dim %d: must be 32..=256, multiple of 32",
                    head_dim);
    return 0;
}

}  // namespace

extern "C" {

int hipml_kv_encode(hipml_stream_t stream, const int *step, int dtype, const float *k_row,
                    const float *v_row, void *k_cache, void *v_cache, int n_kv, int head_dim,
                    int stride) {
    if (int e = check_encode(dtype, n_kv, head_dim, stride)) return e;
    void *args[] = {&k_row, &v_row, &k_cache, &v_cache, &head_dim, &stride, &step};
    return launch_pdl_args(lookup_kv_kernel(dtype == 1 ? "kv_encode_q4" : "kv_encode_q8"), dim3(n_kv),
                           dim3(head_dim), args, 0, as_stream(stream));
}

int hipml_kv_encode_bulk(hipml_stream_t stream, int dtype, const float *k_f32, const float *v_f32,
                         void *k_cache, void *v_cache, int n_kv, int head_dim, int stride,
                         int start, int src0, int rows) {
    if (int e = check_encode(dtype, n_kv, head_dim, stride)) return e;
    if (rows < 0 || start < 0 || src0 < 0 || start + rows > stride)
        return fail(HIPML_ERR_INVALID_ARGUMENT, "rows [%d, %d) beyond KV cache %d", start,
                    start + rows, stride);
    if (rows == 0) return 0;
    if (head_dim == 256 && ((reinterpret_cast<size_t>(k_f32) | reinterpret_cast<size_t>(v_f32)) & 15) == 0)
        return (dtype == 1 ? launch_kv_encode_bulk_rows_q4 : launch_kv_encode_bulk_rows)(
            as_stream(stream), k_f32, v_f32, (unsigned char *)k_cache, (unsigned char *)v_cache, n_kv,
            stride, start, src0, rows);
    // Any other head_dim or alignment: the kernel with the reference's launch shape, one CTA
    // per (row, head) pair up to a few waves of the device; the kernel strides.
    const long long pairs = (long long)n_kv * rows;
    const unsigned grid = (unsigned)(pairs < 148LL * 64 ? pairs : 148LL * 64);
    void *args[] = {&k_f32, &v_f32, &k_cache, &v_cache, &n_kv, &head_dim, &stride, &start, &rows,
                    &src0};
    return launch_pdl_args(lookup_kv_kernel(dtype == 1 ? "kv_encode_bulk_q4" : "kv_encode_bulk_q8"),
                           dim3(grid), dim3(head_dim), args, 0, as_stream(stream));
}

int hipml_kv_encode_rows(hipml_stream_t stream, int dtype, const float *k_f32, const float *v_f32,
                         void *k_cache, void *v_cache, int n_kv, int head_dim, int stride,
                         const int *pos, int slot_bytes, int slots) {
    if (int e = check_encode(dtype, n_kv, head_dim, stride)) return e;
    if (slots <= 0) return fail(HIPML_ERR_INVALID_ARGUMENT, "slots %d must be positive", slots);
    void *args[] = {&k_f32, &v_f32, &k_cache, &v_cache, &n_kv, &head_dim, &stride, &pos,
                    &slot_bytes};
    return launch_pdl_args(lookup_kv_kernel(dtype == 1 ? "kv_encode_q4_b" : "kv_encode_q8_b"),
                           dim3(n_kv, slots), dim3(head_dim), args, 0, as_stream(stream));
}

int hipml_kv_append_f32(hipml_stream_t stream, const int *step, float *k_cache, float *v_cache,
                        const float *k_row, const float *v_row, int width) {
    if (width <= 0) return fail(HIPML_ERR_INVALID_ARGUMENT, "width %d must be positive", width);
    void *args[] = {&k_cache, &v_cache, &k_row, &v_row, &step, &width};
    return (int)cudaLaunchKernel(lookup_kv_kernel("kv_append_f32"), dim3((2 * width + 255) / 256),
                                 dim3(256), args, 0, as_stream(stream));
}

int hipml_kv_append_chunk_f32(hipml_stream_t stream, float *k_cache, float *v_cache,
                              const float *k, const float *v, int pos0, int width, int tokens) {
    if (width <= 0 || tokens < 0 || pos0 < 0)
        return fail(HIPML_ERR_INVALID_ARGUMENT, "width %d / tokens %d / pos0 %d", width, tokens, pos0);
    if (tokens == 0) return 0;
    const long long n = (long long)tokens * width;
    long long blocks = (n / 4 + 255) / 256;
    if (blocks < 1) blocks = 1;
    if (blocks > 148 * 16) blocks = 148 * 16;
    void *args[] = {&k_cache, &v_cache, &k, &v, &pos0, &width, &tokens};
    return (int)cudaLaunchKernel(lookup_kv_kernel("kv_append_chunk_f32"), dim3((unsigned)blocks),
                                 dim3(256), args, 0, as_stream(stream));
}

// Peer-memory exchange that replaces the plain fold (hipml_attn_decode_kv_shard_exchange).
struct ExchangeArgs {
    void *const *peer_ws;
    int shards, rank, phases;
    unsigned wait_limit_us;
    int by_head;
};

static int decode_kv(hipml_stream_t stream, const int *step, int selector, const float *q,
                     const void *k, const void *v, float *part_acc, float *part_ml, float *out,
                     int n_heads, int n_kv, int head_dim, int stride, float scale, int splits,
                     size_t k_off, size_t v_off, bool shard, const ExchangeArgs *xch = nullptr,
                     const float *gate = nullptr, const float *k_row = nullptr,
                     const float *v_row = nullptr) {
    if (int e = check_heads(n_heads, n_kv, head_dim)) return e;
    // The reference remaps selector 0 to its warp kernel at head_dim 256; ids it keeps for
    // experimental variants have no counterpart here.
    bool tensor_core;
    if (selector == 0 || selector == 4 || selector == 7 || selector == 8) {
        // (7 / 8: this library's two bodies by name -- values on mma.sync / on tcgen05 kind::i8 --
        // for A/B runs, head_dim 256 only; 0 takes the process-wide default)
        tensor_core = head_dim == 256;
        if (selector != 0 && head_dim != 256)
            return fail(HIPML_ERR_INVALID_ARGUMENT,
                        "head_dim %d: the warp kernel is head_dim 256 only", head_dim);
    } else if (selector == 6) {
        tensor_core = false;
    } else if (selector == 1) {
        // q4_0: the same tile kernel reading the 144-byte rows in place, at head_dim 256
        tensor_core = head_dim == 256;
    } else {
        return fail(HIPML_ERR_INVALID_ARGUMENT, "unknown KV dtype %d", selector);
    }
    if (splits < 1) splits = 1;
    if (stride <= 0) return fail(HIPML_ERR_INVALID_ARGUMENT, "stride %d must be positive", stride);
    if (((k_off | v_off) & 15) != 0)
        return fail(HIPML_ERR_INVALID_ARGUMENT, "k_off/v_off must be multiples of 16 bytes");
    DecodeParams p;
    p.q = q;
    p.k = (const unsigned char *)k + k_off;
    p.v = (const unsigned char *)v + v_off;
    p.part_acc = part_acc;
    p.part_ml = part_ml;
    p.len = step;
    p.len_stride = 0;
    p.len_offset = 1;
    p.n_heads = n_heads;
    p.n_kv = n_kv;
    p.head_dim = head_dim;
    p.stride = stride;
    p.scale_log2 = scale * kLog2e;
    p.splits = splits;
    p.by_stride = 0;
    p.q4 = selector == 1;
    p.legacy_body = selector == 7 ? 1 : (selector == 8 ? 2 : 0);
    p.run_cap = decode_run_cap(n_kv);
    p.share_slots = 0;
    p.n_slots = 1;
    p.kv_slot_bytes = p.acc_slot = p.ml_slot = p.q_slot = 0;
    if (tensor_core && ((reinterpret_cast<size_t>(p.k) | reinterpret_cast<size_t>(p.v)) & 15) != 0)
        return fail(HIPML_ERR_INVALID_ARGUMENT, "the KV cache must be 16-byte aligned");
    if (tensor_core && (reinterpret_cast<size_t>(q) & 7) != 0)
        return fail(HIPML_ERR_INVALID_ARGUMENT, "the query row must be 8-byte aligned");
    if (k_row) {
        // the caller checked that this combination has the fused form
        p.k_row = k_row;
        p.v_row = v_row;
        p.kw = const_cast<unsigned char *>(p.k);
        p.vw = const_cast<unsigned char *>(p.v);
        p.row_slot = 0;
    }
    if (tensor_core) {
        // one launch: the split pass folds its own partials (and runs the exchange)
        const size_t align = reinterpret_cast<size_t>(out) | reinterpret_cast<size_t>(gate) |
                             reinterpret_cast<size_t>(part_acc);
        if (align & (shard && !xch ? 7 : 15))
            return fail(HIPML_ERR_INVALID_ARGUMENT, "out, gate and part_acc must be 16-byte aligned");
        if ((reinterpret_cast<size_t>(part_ml) & 7) != 0)
            return fail(HIPML_ERR_INVALID_ARGUMENT, "part_ml must be 8-byte aligned");
        p.out = out;
        p.out_slot = 0;
        p.out_head_stride = (shard && !xch) ? head_dim + 2 : head_dim;
        p.normalize = (shard && !xch) ? 0 : 1;
        p.gate = gate;
        if (xch) {
            for (int w = 0; w < 16; w++)
                p.xch.ws[w] = w < xch->shards ? reinterpret_cast<unsigned char *>(xch->peer_ws[w]) : nullptr;
            p.xch.shards = xch->shards;
            p.xch.rank = xch->rank;
            p.xch.phases = xch->phases;
            p.xch.wait_us = xch->wait_limit_us;
            p.xch.by_head = xch->by_head;
            // (divided by head a CTA publishes each of its heads once, to its owner: the split
            // pass does that itself at any rank count)
            if (xch->shards > kInKernelShards && xch->phases == 3 && !xch->by_head) {
                // many ranks: the split pass leaves the folded triples in the workspace's staging
                // rows and a grid of (head, rank) CTAs does the exchange
                DecodeParams local = p;
                local.xch.phases = 0;
                local.out = decode_exchange_stage(xch->peer_ws[xch->rank], n_heads, xch->shards);
                local.out_head_stride = head_dim + 2;
                local.normalize = 0;
                local.gate = nullptr;
                if (int e = launch_decode_tc(as_stream(stream), local, 1)) return e;
                int *status = device_status_word();
                if (!status) return launch_status();
                return launch_decode_exchange_wide(as_stream(stream), p, status);
            }
        }
        return launch_decode_tc(as_stream(stream), p, 1);
    }
    if (xch)
        return fail(HIPML_ERR_INVALID_ARGUMENT,
                    "exchange: only the head_dim 256 kernel (selectors 0, 1, 4) publishes to peers");
    if (int e = launch_decode_split(as_stream(stream), p, 1, false)) return e;
    if (!shard)
        return launch_decode_reduce(as_stream(stream), part_acc, part_ml, out, n_heads, head_dim,
                                    splits, 1, 0, 0, 0, gate);
    FoldParams f;
    f.acc = part_acc;
    f.ml = part_ml;
    f.out = out;
    f.head_dim = head_dim;
    f.splits = splits;
    f.acc_head_stride = (long long)splits * head_dim;
    f.acc_split_stride = head_dim;
    f.ml_head_stride = (long long)splits * 2;
    f.ml_split_stride = 2;
    f.acc_slot = f.ml_slot = f.out_slot = 0;
    f.out_head_stride = head_dim + 2;
    f.normalize = 0;
    f.gate = nullptr;
    return launch_decode_fold(as_stream(stream), f, n_heads, 1);
}

int hipml_attn_decode_kv(hipml_stream_t stream, const int *step, int selector, const float *q,
                         const void *k, const void *v, float *part_acc, float *part_ml,
                         float *out, int n_heads, int n_kv, int head_dim, int stride, float scale,
                         int splits, size_t k_off, size_t v_off) {
    return decode_kv(stream, step, selector, q, k, v, part_acc, part_ml, out, n_heads, n_kv,
                     head_dim, stride, scale, splits, k_off, v_off, false);
}

int hipml_attn_decode_kv_gated(hipml_stream_t stream, const int *step, int selector, const float *q,
                               const void *k, const void *v, float *part_acc, float *part_ml,
                               float *out, const float *gate, int n_heads, int n_kv, int head_dim,
                               int stride, float scale, int splits, size_t k_off, size_t v_off) {
    if (!gate) return fail(HIPML_ERR_INVALID_ARGUMENT, "gated decode: no gate row");
    return decode_kv(stream, step, selector, q, k, v, part_acc, part_ml, out, n_heads, n_kv,
                     head_dim, stride, scale, splits, k_off, v_off, false, nullptr, gate);
}

int hipml_attn_decode_kv_append(hipml_stream_t stream, const int *step, int selector,
                                const float *k_row, const float *v_row, const float *q, void *k,
                                void *v, float *part_acc, float *part_ml, float *out,
                                const float *gate, int n_heads, int n_kv, int head_dim, int stride,
                                float scale, int splits, size_t k_off, size_t v_off) {
    if (!k_row || !v_row) return fail(HIPML_ERR_INVALID_ARGUMENT, "decode with append: no K/V row");
    if (((k_off | v_off) & 15) != 0)
        return fail(HIPML_ERR_INVALID_ARGUMENT, "k_off/v_off must be multiples of 16 bytes");
    unsigned char *kc = (unsigned char *)k + k_off, *vc = (unsigned char *)v + v_off;
    const bool fused =
        (selector == 0 || selector == 1 || selector == 4 || selector == 7 || selector == 8) && head_dim == 256 &&
        ((reinterpret_cast<size_t>(kc) | reinterpret_cast<size_t>(vc) | reinterpret_cast<size_t>(k_row) |
          reinterpret_cast<size_t>(v_row)) & 15) == 0;
    if (!fused) {
        // any other selector, head size or alignment: the two launches the reference makes
        const int dtype = selector == 1 ? 1 : 0;
        if (selector != 0 && selector != 1 && selector != 4 && selector != 6 && selector != 7 && selector != 8)
            return fail(HIPML_ERR_INVALID_ARGUMENT, "unknown KV dtype %d", selector);
        if (int e = hipml_kv_encode(stream, step, dtype, k_row, v_row, kc, vc, n_kv, head_dim, stride))
            return e;
        return decode_kv(stream, step, selector, q, k, v, part_acc, part_ml, out, n_heads, n_kv,
                         head_dim, stride, scale, splits, k_off, v_off, false, nullptr, gate);
    }
    return decode_kv(stream, step, selector, q, k, v, part_acc, part_ml, out, n_heads, n_kv,
                     head_dim, stride, scale, splits, k_off, v_off, false, nullptr, gate, k_row, v_row);
}

int hipml_attn_decode_kv_shard(hipml_stream_t stream, const int *step, int selector,
                               const float *q, const void *k, const void *v, float *part_acc,
                               float *part_ml, float *shard_out, int n_heads, int n_kv,
                               int head_dim, int stride, float scale, int splits, size_t k_off,
                               size_t v_off) {
    return decode_kv(stream, step, selector, q, k, v, part_acc, part_ml, shard_out, n_heads, n_kv,
                     head_dim, stride, scale, splits, k_off, v_off, true);
}

size_t hipml_decode_exchange_bytes(int n_heads, int head_dim, int shards) {
    if (n_heads <= 0 || head_dim <= 0 || shards <= 0) return 0;
    return decode_exchange_bytes(n_heads, head_dim, shards);
}

static int shard_exchange(hipml_stream_t stream, const int *step, int selector, const float *k_row,
                          const float *v_row, const float *q, const void *k, const void *v,
                          float *part_acc, float *part_ml, float *out, int n_heads, int n_kv,
                          int head_dim, int stride, float scale, int splits, size_t k_off,
                          size_t v_off, void *const *peer_ws, int shards, int rank, int phases,
                          unsigned wait_limit_us) {
    if (shards < 1 || shards > 16 || rank < 0 || rank >= shards)
        return fail(HIPML_ERR_INVALID_ARGUMENT, "exchange: rank %d of %d shards (1..16)", rank,
                    shards);
    const int by_head = (phases >> 2) & 1;
    phases &= ~4;
    if (phases < 1 || phases > 3)
        return fail(HIPML_ERR_INVALID_ARGUMENT,
                    "exchange: phases %d (1 publish, 2 collect, 3 both; + 4 result divided by head)", phases);
    if (by_head && (n_heads <= 0 || n_heads % shards != 0))
        return fail(HIPML_ERR_INVALID_ARGUMENT, "exchange by head: %d heads over %d ranks", n_heads, shards);
    if (!peer_ws) return fail(HIPML_ERR_INVALID_ARGUMENT, "exchange: no workspace table");
    for (int w = 0; w < shards; w++)
        if (!peer_ws[w] || (reinterpret_cast<size_t>(peer_ws[w]) & 255) != 0)
            return fail(HIPML_ERR_WORKSPACE, "exchange: workspace %d missing or not 256-byte aligned", w);
    if (head_dim != 256)
        return fail(HIPML_ERR_INVALID_ARGUMENT, "exchange: head_dim %d, only 256", head_dim);
    if (wait_limit_us > 10000000u) wait_limit_us = 10000000u;
    ExchangeArgs x = {peer_ws, shards, rank, phases, wait_limit_us, by_head};
    if (phases == 2) {
        // collect only: no split pass, the partials are not read
        if (int e = check_heads(n_heads, n_kv, head_dim)) return e;
        if ((reinterpret_cast<size_t>(out) & 15) != 0)
            return fail(HIPML_ERR_INVALID_ARGUMENT, "out, gate and part_acc must be 16-byte aligned");
        int *status = device_status_word();
        if (!status) return launch_status();
        DecodeParams p = {};
        p.n_heads = n_heads;
        p.n_kv = n_kv;
        p.head_dim = head_dim;
        p.out = out;
        p.out_slot = 0;
        p.out_head_stride = head_dim;
        p.normalize = 1;
        for (int w = 0; w < 16; w++)
            p.xch.ws[w] = w < shards ? reinterpret_cast<unsigned char *>(peer_ws[w]) : nullptr;
        p.xch.shards = shards;
        p.xch.rank = rank;
        p.xch.phases = 2;
        p.xch.wait_us = wait_limit_us;
        p.xch.by_head = by_head;
        return launch_decode_collect(as_stream(stream), p, status);
    }
    if (k_row &&
        ((reinterpret_cast<size_t>(k_row) | reinterpret_cast<size_t>(v_row)) & 15) != 0)
        return fail(HIPML_ERR_INVALID_ARGUMENT, "decode with append: K/V rows must be 16-byte aligned");
    return decode_kv(stream, step, selector, q, k, v, part_acc, part_ml, out, n_heads, n_kv,
                     head_dim, stride, scale, splits, k_off, v_off, true, &x, nullptr, k_row, v_row);
}

int hipml_attn_decode_kv_shard_exchange(hipml_stream_t stream, const int *step, int selector,
                                        const float *q, const void *k, const void *v,
                                        float *part_acc, float *part_ml, float *out, int n_heads,
                                        int n_kv, int head_dim, int stride, float scale, int splits,
                                        size_t k_off, size_t v_off, void *const *peer_ws,
                                        int shards, int rank, int phases,
                                        unsigned wait_limit_us) {
    return shard_exchange(stream, step, selector, nullptr, nullptr, q, k, v, part_acc, part_ml, out,
                          n_heads, n_kv, head_dim, stride, scale, splits, k_off, v_off, peer_ws, shards,
                          rank, phases, wait_limit_us);
}

int hipml_attn_decode_kv_shard_exchange_append(hipml_stream_t stream, const int *step, int selector,
                                               const float *k_row, const float *v_row,
                                               const float *q, void *k, void *v, float *part_acc,
                                               float *part_ml, float *out, int n_heads, int n_kv,
                                               int head_dim, int stride, float scale, int splits,
                                               size_t k_off, size_t v_off, void *const *peer_ws,
                                               int shards, int rank, int phases,
                                               unsigned wait_limit_us) {
    if ((k_row == nullptr) != (v_row == nullptr))
        return fail(HIPML_ERR_INVALID_ARGUMENT, "decode with append: give both rows or neither");
    return shard_exchange(stream, step, selector, k_row, v_row, q, k, v, part_acc, part_ml, out,
                          n_heads, n_kv, head_dim, stride, scale, splits, k_off, v_off, peer_ws, shards,
                          rank, phases, wait_limit_us);
}

int hipml_attn_decode_combine(hipml_stream_t stream, const float *gathered, float *out,
                              int n_heads, int head_dim, int shards) {
    if (n_heads <= 0 || shards <= 0 || head_dim % 32 != 0 || head_dim < 32 || head_dim > 256)
        return fail(HIPML_ERR_INVALID_ARGUMENT, "combine: n_heads %d / head_dim %d / shards %d",
                    n_heads, head_dim, shards);
    FoldParams f;
    f.acc = gathered;
    f.ml = gathered + head_dim;
    f.out = out;
    f.head_dim = head_dim;
    f.splits = shards;
    f.acc_head_stride = f.ml_head_stride = head_dim + 2;
    f.acc_split_stride = f.ml_split_stride = (long long)n_heads * (head_dim + 2);
    f.acc_slot = f.ml_slot = f.out_slot = 0;
    f.out_head_stride = head_dim;
    f.normalize = 1;
    f.gate = nullptr;
    return launch_decode_fold(as_stream(stream), f, n_heads, 1);
}

static int decode_rows(hipml_stream_t stream, int dtype, const int *pos, const float *q,
                       const void *k_cache, const void *v_cache, float *part_acc, float *part_ml,
                       float *out, int n_heads, int n_kv, int head_dim, int stride, float scale,
                       int splits, int kv_slot_bytes, int acc_slot, int ml_slot, int q_slot,
                       int slots, int by_stride, const float *k_rows = nullptr,
                       const float *v_rows = nullptr) {
    if (int e = check_heads(n_heads, n_kv, head_dim)) return e;
    if (dtype != 0 && dtype != 1)
        return fail(HIPML_ERR_INVALID_ARGUMENT, "unknown KV dtype %d", dtype);
    if (slots <= 0 || splits < 1 || stride <= 0)
        return fail(HIPML_ERR_INVALID_ARGUMENT, "slots %d / splits %d / stride %d", slots, splits,
                    stride);
    DecodeParams p;
    p.q = q;
    p.k = (const unsigned char *)k_cache;
    p.v = (const unsigned char *)v_cache;
    p.part_acc = part_acc;
    p.part_ml = part_ml;
    p.len = pos;
    p.len_stride = 2;
    p.len_offset = 1;
    p.n_heads = n_heads;
    p.n_kv = n_kv;
    p.head_dim = head_dim;
    p.stride = stride;
    p.scale_log2 = scale * kLog2e;
    p.splits = splits;
    p.by_stride = by_stride;
    p.q4 = dtype == 1;
    p.n_slots = slots;
    p.run_cap = by_stride ? 0 : decode_run_cap(n_kv);
    // Several slots of unequal depth: the slots share one round of CTAs in proportion to their
    // live lengths (every CTA reads all the lengths, so only for a moderate number of slots);
    // the fixed cache-position runs remain for the kernels without this plan.
    p.share_slots =
        (by_stride && slots > 1 && slots <= 64 && 2 * slots * n_kv <= decode_cta_slots()) ? decode_cta_slots()
                                                                                          : 0;
    p.kv_slot_bytes = kv_slot_bytes;
    p.acc_slot = acc_slot;
    p.ml_slot = ml_slot;
    p.q_slot = q_slot;
    const bool aligned =
        ((reinterpret_cast<size_t>(p.k) | reinterpret_cast<size_t>(p.v) | (size_t)kv_slot_bytes) &
         15) == 0;
    const bool tensor_core = head_dim == 256 && aligned && (reinterpret_cast<size_t>(q) & 7) == 0 &&
                             (q_slot & 1) == 0;
    if (k_rows) {
        // fused append (the caller checked that this combination has it)
        if (!tensor_core)
            return fail(HIPML_ERR_INVALID_ARGUMENT, "decode with append: no fused form for this shape");
        p.k_row = k_rows;
        p.v_row = v_rows;
        p.kw = const_cast<unsigned char *>(p.k);
        p.vw = const_cast<unsigned char *>(p.v);
        p.row_slot = (long long)n_kv * head_dim;
    }
    // The tensor-core body folds its own partials (groups of eight runs, then the groups: at
    // most 32 groups), unless the fixed runs of a very fine caller plan are too many for that.
    const bool fixed_runs = p.share_slots == 0 && (by_stride || p.run_cap <= 0);
    const bool tree = tensor_core && !(fixed_runs && splits > 256) &&
                      ((reinterpret_cast<size_t>(out) | reinterpret_cast<size_t>(part_acc)) & 15) == 0 &&
                      (reinterpret_cast<size_t>(part_ml) & 7) == 0 && ((acc_slot | q_slot) & 3) == 0 &&
                      (ml_slot & 1) == 0;
    if (tree) {
        p.out = out;
        p.out_slot = q_slot;
        p.out_head_stride = head_dim;
        p.normalize = 1;
        return launch_decode_tc(as_stream(stream), p, slots);
    }
    if (tensor_core && !fixed_runs) {
        // only the live runs of the device's plan are written; the flat fold reads all `splits`
        p.run_cap = 0;
        p.share_slots = 0;
        p.by_stride = by_stride;
    }
    if (int e = launch_decode_split(as_stream(stream), p, slots, tensor_core)) return e;
    return launch_decode_reduce(as_stream(stream), part_acc, part_ml, out, n_heads, head_dim, splits,
                                slots, acc_slot, ml_slot, q_slot, nullptr);
}

int hipml_attn_decode_rows(hipml_stream_t stream, int dtype, const int *pos, const float *q,
                           const void *k_cache, const void *v_cache, float *part_acc,
                           float *part_ml, float *out, int n_heads, int n_kv, int head_dim,
                           int stride, float scale, int splits, int kv_slot_bytes, int acc_slot,
                           int ml_slot, int q_slot, int slots) {
    return decode_rows(stream, dtype, pos, q, k_cache, v_cache, part_acc, part_ml, out, n_heads,
                       n_kv, head_dim, stride, scale, splits, kv_slot_bytes, acc_slot, ml_slot,
                       q_slot, slots, 1);
}

int hipml_attn_decode_cols(hipml_stream_t stream, int selector, const int *pos, const float *q,
                           const void *k, const void *v, float *part_acc, float *part_ml,
                           float *out, int n_heads, int n_kv, int head_dim, int stride, float scale,
                           int splits, int cols, int acc_slot, int ml_slot, int q_slot) {
    if (selector != 0 && selector != 4)
        return fail(HIPML_ERR_INVALID_ARGUMENT, "decode columns: selector %d has no batched entry",
                    selector);
    // The columns share the cache (no slot offset) and each is partitioned over its own live
    // length, exactly as its one-column launch would be.
    return decode_rows(stream, 0, pos, q, k, v, part_acc, part_ml, out, n_heads, n_kv, head_dim,
                       stride, scale, splits, 0, acc_slot, ml_slot, q_slot, cols, 0);
}

int hipml_kv_rows_copy(hipml_stream_t stream, void *dst, const void *src, int n_kv, int row_bytes,
                       int dst_stride, int src_stride, int rows) {
    if (n_kv <= 0 || row_bytes <= 0 || rows < 0 || rows > dst_stride || rows > src_stride)
        return fail(HIPML_ERR_INVALID_ARGUMENT,
                    "rows copy: n_kv %d / row_bytes %d / rows %d of strides %d, %d", n_kv, row_bytes,
                    rows, dst_stride, src_stride);
    if (rows == 0) return 0;
    // one contiguous run of rows * row_bytes per KV head
    return (int)cudaMemcpy2DAsync(dst, (size_t)dst_stride * row_bytes, src,
                                  (size_t)src_stride * row_bytes, (size_t)rows * row_bytes, n_kv,
                                  cudaMemcpyDeviceToDevice, as_stream(stream));
}

int hipml_attn_decode_batch(hipml_stream_t stream, int dtype, const int *pos, const float *q,
                            const void *k_cache, const void *v_cache, float *part_acc,
                            float *part_ml, float *out, int n_heads, int n_kv, int head_dim,
                            int stride, float scale, int splits, int kv_slot_bytes, int acc_slot,
                            int ml_slot, int q_slot, int slots, int live_seq) {
    if (n_kv <= 0 || n_heads % n_kv != 0)
        return fail(HIPML_ERR_INVALID_ARGUMENT, "n_heads %d is not a multiple of n_kv %d", n_heads,
                    n_kv);
    const int group = n_heads / n_kv;
    const bool one = live_seq > 0 && slots == 1 && dtype == 0 && head_dim == 256 && group <= 8;
    if (one) {
        // A lone slot partitions over its live length, as the single-stream engine does.
        int live = live_seq / 32;
        live = live < 1 ? 1 : (live > 256 ? 256 : live);
        if (live > splits) live = splits;
        return decode_rows(stream, dtype, pos, q, k_cache, v_cache, part_acc, part_ml, out,
                           n_heads, n_kv, head_dim, stride, scale, live, kv_slot_bytes, acc_slot,
                           ml_slot, q_slot, 1, 0);
    }
    return decode_rows(stream, dtype, pos, q, k_cache, v_cache, part_acc, part_ml, out, n_heads,
                       n_kv, head_dim, stride, scale, splits, kv_slot_bytes, acc_slot, ml_slot,
                       q_slot, slots, 1);
}

int hipml_attn_decode_batch_append(hipml_stream_t stream, int dtype, const int *pos,
                                   const float *k_f32, const float *v_f32, const float *q,
                                   void *k_cache, void *v_cache, float *part_acc, float *part_ml,
                                   float *out, int n_heads, int n_kv, int head_dim, int stride,
                                   float scale, int splits, int kv_slot_bytes, int acc_slot,
                                   int ml_slot, int q_slot, int slots) {
    if (!k_f32 || !v_f32) return fail(HIPML_ERR_INVALID_ARGUMENT, "decode with append: no K/V rows");
    const bool fused =
        (dtype == 0 || dtype == 1) && head_dim == 256 && slots > 0 &&
        ((reinterpret_cast<size_t>(k_cache) | reinterpret_cast<size_t>(v_cache) | (size_t)kv_slot_bytes |
          reinterpret_cast<size_t>(k_f32) | reinterpret_cast<size_t>(v_f32)) & 15) == 0;
    if (!fused) {
        if (int e = hipml_kv_encode_rows(stream, dtype, k_f32, v_f32, k_cache, v_cache, n_kv, head_dim,
                                         stride, pos, kv_slot_bytes, slots))
            return e;
        return decode_rows(stream, dtype, pos, q, k_cache, v_cache, part_acc, part_ml, out, n_heads,
                           n_kv, head_dim, stride, scale, splits, kv_slot_bytes, acc_slot, ml_slot,
                           q_slot, slots, 1);
    }
    return decode_rows(stream, dtype, pos, q, k_cache, v_cache, part_acc, part_ml, out, n_heads, n_kv,
                       head_dim, stride, scale, splits, kv_slot_bytes, acc_slot, ml_slot, q_slot,
                       slots, 1, k_f32, v_f32);
}

size_t hipml_attn_chunk_workspace_bytes(int n_kv, int head_dim, int pos0, int tokens) {
    if (head_dim != 256 || n_kv <= 0 || pos0 < 0 || tokens <= 0) return 0;
    return chunk_tc_workspace_bytes(n_kv, pos0 + tokens);
}

int hipml_attn_chunk(hipml_stream_t stream, const float *q, const void *k_cache,
                     const void *v_cache, float *out, int n_heads, int n_kv, int head_dim,
                     int pos0, int tokens, int kv_dtype, int stride, float *part_acc,
                     float *part_ml, int splits, int mode, void *workspace,
                     size_t workspace_bytes) {
    if (n_kv <= 0 || n_heads % n_kv != 0)
        return fail(HIPML_ERR_INVALID_ARGUMENT, "n_heads %d is not a multiple of n_kv %d", n_heads,
                    n_kv);
    const int group = n_heads / n_kv;
    if (kv_dtype < 0 || kv_dtype > 2)
        return fail(HIPML_ERR_INVALID_ARGUMENT, "unknown KV dtype %d", kv_dtype);
    if (kv_dtype != 0 && !(head_dim == 256 && group <= 8))
        return fail(HIPML_ERR_INVALID_ARGUMENT, "quantized chunk attention: unsupported shape");
    if (head_dim % 32 != 0 || head_dim < 32 || head_dim > 256)
        return fail(HIPML_ERR_INVALID_ARGUMENT, "head_dim %d: must be 32..=256, multiple of 32",
                    head_dim);
    if (pos0 < 0 || tokens < 0)
        return fail(HIPML_ERR_INVALID_ARGUMENT, "pos0 %d / tokens %d", pos0, tokens);
    if (kv_dtype != 0 && pos0 + tokens > stride)
        return fail(HIPML_ERR_INVALID_ARGUMENT, "position %d beyond KV cache %d", pos0 + tokens,
                    stride);
    if (mode < 0 || mode > 3) return fail(HIPML_ERR_INVALID_ARGUMENT, "unknown mode %d", mode);
    if (tokens == 0) return 0;
    if (splits >= 2 && (!part_acc || !part_ml))
        return fail(HIPML_ERR_INVALID_ARGUMENT, "split attention needs part_acc and part_ml");
    const int qslots = (tokens + 31) / 32 * 32;
    const float scale = 1.0f / sqrtf((float)head_dim);

    if (mode == 2) {
        ChunkScalarParams p;
        p.q = q;
        p.k = k_cache;
        p.v = v_cache;
        p.out = out;
        p.part_acc = part_acc;
        p.part_ml = part_ml;
        p.n_heads = n_heads;
        p.n_kv = n_kv;
        p.head_dim = head_dim;
        p.pos0 = pos0;
        p.tokens = tokens;
        p.kv_dtype = kv_dtype;
        p.stride = stride;
        p.scale_log2 = scale * kLog2e;
        p.splits = splits;
        p.qslots = qslots;
        if (int e = launch_chunk_scalar(as_stream(stream), p)) return e;
    } else {
        if (head_dim != 256 || group > 8)
            return fail(HIPML_ERR_INVALID_ARGUMENT,
                        "tensor-core chunk attention: only head_dim 256 with a GQA group <= 8");
        const int cap = (pos0 + tokens + 127) / 128 * 128;
        if (int e = hipml_attn_chunk_stage(stream, k_cache, v_cache, n_kv, head_dim, kv_dtype,
                                           stride, 0, pos0 + tokens, cap, workspace,
                                           workspace_bytes))
            return e;
        return hipml_attn_chunk_staged(stream, q, out, n_heads, n_kv, head_dim, pos0, tokens,
                                       part_acc, part_ml, splits, mode, cap, workspace,
                                       workspace_bytes);
    }
    if (splits >= 2)
        return launch_chunk_combine(as_stream(stream), part_acc, part_ml, out, n_heads, head_dim,
                                    tokens, qslots, splits);
    return 0;
}

int hipml_attn_chunk_stage(hipml_stream_t stream, const void *k_cache, const void *v_cache,
                           int n_kv, int head_dim, int kv_dtype, int stride, int key_from,
                           int key_to, int key_capacity, void *workspace,
                           size_t workspace_bytes) {
    if (head_dim != 256 || n_kv <= 0)
        return fail(HIPML_ERR_INVALID_ARGUMENT,
                    "tensor-core chunk attention: only head_dim 256 with a GQA group <= 8");
    if (kv_dtype < 0 || kv_dtype > 2)
        return fail(HIPML_ERR_INVALID_ARGUMENT, "unknown KV dtype %d", kv_dtype);
    if (key_from < 0 || key_to < key_from || key_capacity % 128 != 0 || key_to > key_capacity)
        return fail(HIPML_ERR_INVALID_ARGUMENT, "stage rows [%d, %d) with capacity %d", key_from,
                    key_to, key_capacity);
    if (kv_dtype != 0 && key_to > stride)
        return fail(HIPML_ERR_INVALID_ARGUMENT, "position %d beyond KV cache %d", key_to, stride);
    const size_t need = chunk_tc_workspace_bytes(n_kv, key_capacity);
    if (!workspace || workspace_bytes < need)
        return fail(HIPML_ERR_WORKSPACE, "chunk attention workspace: %zu bytes given, %zu needed",
                    workspace_bytes, need);
    if ((reinterpret_cast<size_t>(workspace) & 255) != 0)
        return fail(HIPML_ERR_WORKSPACE, "chunk attention workspace must be 256-byte aligned");
    if (((reinterpret_cast<size_t>(k_cache) | reinterpret_cast<size_t>(v_cache)) & 15) != 0)
        return fail(HIPML_ERR_INVALID_ARGUMENT, "q, out and the caches must be 16-byte aligned");
    return launch_chunk_stage(as_stream(stream), k_cache, v_cache, n_kv, kv_dtype, stride, key_from,
                              key_to, key_capacity, workspace);
}

static int chunk_staged(hipml_stream_t stream, const float *q, float *out, int n_heads, int n_kv,
                        int head_dim, int pos0, int tokens, float *part_acc, float *part_ml,
                        int splits, int mode, int key_capacity, void *workspace,
                        size_t workspace_bytes, const float *gate) {
    if (n_kv <= 0 || n_heads % n_kv != 0)
        return fail(HIPML_ERR_INVALID_ARGUMENT, "n_heads %d is not a multiple of n_kv %d", n_heads,
                    n_kv);
    if (head_dim != 256 || n_heads / n_kv > 8)
        return fail(HIPML_ERR_INVALID_ARGUMENT,
                    "tensor-core chunk attention: only head_dim 256 with a GQA group <= 8");
    if (mode != 0 && mode != 1 && mode != 3)
        return fail(HIPML_ERR_INVALID_ARGUMENT, "unknown mode %d", mode);
    if (pos0 < 0 || tokens < 0 || key_capacity % 128 != 0 || pos0 + tokens > key_capacity)
        return fail(HIPML_ERR_INVALID_ARGUMENT, "rows [%d, %d) with capacity %d", pos0,
                    pos0 + tokens, key_capacity);
    if (tokens == 0) return 0;
    if (splits >= 2 && (!part_acc || !part_ml))
        return fail(HIPML_ERR_INVALID_ARGUMENT, "split attention needs part_acc and part_ml");
    if (splits >= 2 && ((reinterpret_cast<size_t>(part_acc) & 15) != 0 || (reinterpret_cast<size_t>(part_ml) & 7) != 0))
        return fail(HIPML_ERR_INVALID_ARGUMENT, "split attention: part_acc must be 16-byte, part_ml 8-byte aligned");
    const size_t need = chunk_tc_workspace_bytes(n_kv, key_capacity);
    if (!workspace || workspace_bytes < need)
        return fail(HIPML_ERR_WORKSPACE, "chunk attention workspace: %zu bytes given, %zu needed",
                    workspace_bytes, need);
    if ((reinterpret_cast<size_t>(workspace) & 255) != 0)
        return fail(HIPML_ERR_WORKSPACE, "chunk attention workspace must be 256-byte aligned");
    if (((reinterpret_cast<size_t>(q) | reinterpret_cast<size_t>(out)) & 15) != 0)
        return fail(HIPML_ERR_INVALID_ARGUMENT, "q, out and the caches must be 16-byte aligned");
    int *status = device_status_word();
    if (!status) return launch_status();
    if (int e = launch_chunk_tc(as_stream(stream), q, out, part_acc, part_ml, n_heads, n_kv, pos0,
                                tokens, key_capacity, splits, mode == 1 ? 1 : (mode == 3 ? 2 : 0), workspace,
                                status, splits >= 2 ? nullptr : gate))
        return e;
    if (splits >= 2)
        return launch_chunk_combine(as_stream(stream), part_acc, part_ml, out, n_heads, head_dim,
                                    tokens, (tokens + 31) / 32 * 32, splits, gate);
    return 0;
}

int hipml_attn_chunk_staged(hipml_stream_t stream, const float *q, float *out, int n_heads,
                            int n_kv, int head_dim, int pos0, int tokens, float *part_acc,
                            float *part_ml, int splits, int mode, int key_capacity,
                            void *workspace, size_t workspace_bytes) {
    return chunk_staged(stream, q, out, n_heads, n_kv, head_dim, pos0, tokens, part_acc, part_ml,
                        splits, mode, key_capacity, workspace, workspace_bytes, nullptr);
}

int hipml_attn_chunk_staged_gated(hipml_stream_t stream, const float *q, float *out,
                                  const float *gate, int n_heads, int n_kv, int head_dim, int pos0,
                                  int tokens, float *part_acc, float *part_ml, int splits, int mode,
                                  int key_capacity, void *workspace, size_t workspace_bytes) {
    if (!gate || (reinterpret_cast<size_t>(gate) & 15) != 0)
        return fail(HIPML_ERR_INVALID_ARGUMENT, "gated chunk attention: gate rows missing or unaligned");
    return chunk_staged(stream, q, out, n_heads, n_kv, head_dim, pos0, tokens, part_acc, part_ml,
                        splits, mode, key_capacity, workspace, workspace_bytes, gate);
}

int hipml_kv_append_cols_f32(hipml_stream_t stream, float *k_cache, float *v_cache,
                             const float *k, const float *v, int pos0, int rows, int width) {
    if (width <= 0 || rows < 0 || pos0 < 0)
        return fail(HIPML_ERR_INVALID_ARGUMENT, "width %d / rows %d / pos0 %d", width, rows, pos0);
    if (rows == 0) return 0;
    const long long n = 2LL * width * rows;
    void *args[] = {&k_cache, &v_cache, &k, &v, &pos0, &rows, &width};
    return (int)cudaLaunchKernel(lookup_cols_kernel("kv_append_cols_f32"),
                                 dim3((unsigned)((n + 255) / 256)), dim3(256), args, 0,
                                 as_stream(stream));
}

// ---- attention front end and tail --------------------------------------------------------

static int check_front(int n_heads, int n_kv, int head_dim, int n_rot) {
    if (n_heads <= 0 || n_kv <= 0 || head_dim <= 0 || head_dim > 256)
        return fail(HIPML_ERR_INVALID_ARGUMENT, "front end: n_heads %d / n_kv %d / head_dim %d (<= 256)",
                    n_heads, n_kv, head_dim);
    if (n_rot < 0 || n_rot > head_dim || n_rot % 2 != 0)
        return fail(HIPML_ERR_INVALID_ARGUMENT, "n_rot must be even and <= head_dim");
    return 0;
}

int hipml_attn_front(hipml_stream_t stream, const float *qg, float *q, float *gate, float *k,
                     const float *q_norm, const float *k_norm, int n_heads, int n_kv, int head_dim,
                     int n_rot, const int *sections, const int *pos, float theta_base, float eps) {
    if (int e = check_front(n_heads, n_kv, head_dim, n_rot)) return e;
    int s0 = sections ? sections[0] : 0, s1 = sections ? sections[1] : 0;
    int s2 = sections ? sections[2] : 0, s3 = sections ? sections[3] : 0;
    void *args[] = {&qg, &q, &gate, &k, &q_norm, &k_norm, &n_heads, &n_kv, &head_dim, &n_rot,
                    &s0, &s1, &s2, &s3, &pos, &theta_base, &eps};
    return launch_pdl_args(lookup_front_kernel("attn_front_f32"), dim3(n_heads + n_kv), dim3(256), args,
                           0, as_stream(stream));
}

int hipml_qg_split_chunk(hipml_stream_t stream, const float *qg, float *q, float *gate, int n_heads,
                         int head_dim, int tokens) {
    if (n_heads <= 0 || head_dim <= 0 || head_dim > 1024 || tokens < 0)
        return fail(HIPML_ERR_INVALID_ARGUMENT, "qg_split: n_heads %d / head_dim %d / tokens %d",
                    n_heads, head_dim, tokens);
    if (tokens == 0) return 0;
    void *args[] = {&qg, &q, &gate, &n_heads, &head_dim, &tokens};
    return launch_pdl_args(lookup_front_kernel("qg_split_chunk_f32"), dim3(n_heads, tokens),
                           dim3(head_dim), args, 0, as_stream(stream));
}

int hipml_norm_rope_chunk(hipml_stream_t stream, float *q, float *k, const float *q_norm,
                          const float *k_norm, int n_heads, int n_kv, int head_dim, int n_rot,
                          float theta_base, float eps, int pos0, int tokens) {
    if (int e = check_front(n_heads, n_kv, head_dim, n_rot)) return e;
    if (head_dim % 32 != 0)
        return fail(HIPML_ERR_INVALID_ARGUMENT, "head_dim %d: must be a multiple of 32", head_dim);
    if (tokens < 0 || pos0 < 0) return fail(HIPML_ERR_INVALID_ARGUMENT, "pos0 %d / tokens %d", pos0, tokens);
    if (tokens == 0) return 0;
    void *args[] = {&q, &k, &q_norm, &k_norm, &n_heads, &n_kv, &head_dim, &n_rot, &theta_base, &eps,
                    &pos0, &tokens};
    return launch_pdl_args(lookup_front_kernel("norm_rope_chunk_f32"), dim3(n_heads + n_kv, tokens),
                           dim3(head_dim), args, 0, as_stream(stream));
}

int hipml_q_gate(hipml_stream_t stream, const float *q, const float *gate, float *y, long long n) {
    if (n < 0) return fail(HIPML_ERR_INVALID_ARGUMENT, "q_gate: n %lld", n);
    return launch_q_gate(as_stream(stream), q, gate, y, n);
}

int hipml_attn_front_append_q8(hipml_stream_t stream, const float *qg, const float *k,
                               const float *v, float *q, float *gate, float *k_out,
                               const float *q_norm, const float *k_norm, void *k_cache,
                               void *v_cache, int n_heads, int n_kv, int head_dim, int n_rot,
                               const int *sections, const int *pos, const int *step, int pos0,
                               int tokens, int stride, float theta_base, float eps) {
    if (int e = check_front(n_heads, n_kv, head_dim, n_rot)) return e;
    if (head_dim != 256 || n_rot % 16 != 0)
        return fail(HIPML_ERR_INVALID_ARGUMENT,
                    "fused front end: head_dim 256 and n_rot a multiple of 16 (got %d, %d)", head_dim,
                    n_rot);
    if (tokens < 0 || pos0 < 0) return fail(HIPML_ERR_INVALID_ARGUMENT, "pos0 %d / tokens %d", pos0, tokens);
    if ((pos || step) && tokens != 1)
        return fail(HIPML_ERR_INVALID_ARGUMENT, "device positions describe one token, got %d", tokens);
    if ((k_cache == nullptr) != (v_cache == nullptr))
        return fail(HIPML_ERR_INVALID_ARGUMENT, "give both caches or neither");
    if (k_cache && (stride <= 0 || (!step && pos0 + tokens > stride)))
        return fail(HIPML_ERR_INVALID_ARGUMENT, "position %d beyond KV cache %d", pos0 + tokens, stride);
    const size_t align = reinterpret_cast<size_t>(qg) | reinterpret_cast<size_t>(k) |
                         reinterpret_cast<size_t>(v) | reinterpret_cast<size_t>(q) |
                         reinterpret_cast<size_t>(gate) | reinterpret_cast<size_t>(k_out) |
                         reinterpret_cast<size_t>(q_norm) | reinterpret_cast<size_t>(k_norm);
    if (align & 15) return fail(HIPML_ERR_INVALID_ARGUMENT, "fused front end: 16-byte aligned rows");
    if (tokens == 0) return 0;
    return launch_front_rows_q8(as_stream(stream), qg, k, v, q, gate, k_out, q_norm, k_norm, k_cache,
                                v_cache, n_heads, n_kv, n_rot, sections, pos, step, pos0, tokens,
                                stride, theta_base, eps);
}

int hipml_attn_decode_cols_f32(hipml_stream_t stream, const float *q, const float *k_cache,
                               const float *v_cache, float *part_acc, float *part_ml, float *out,
                               int n_heads, int n_kv, int head_dim, int n_ctx, int pos0,
                               int rows) {
    if (int e = check_heads(n_heads, n_kv, head_dim)) return e;
    if (n_ctx <= 0 || pos0 < 0 || rows < 0)
        return fail(HIPML_ERR_INVALID_ARGUMENT, "n_ctx %d / pos0 %d / rows %d", n_ctx, pos0, rows);
    if (pos0 + rows > n_ctx)
        return fail(HIPML_ERR_INVALID_ARGUMENT, "position %d beyond KV cache %d", pos0 + rows, n_ctx);
    if (rows == 0) return 0;
    if (!part_acc || !part_ml)
        return fail(HIPML_ERR_INVALID_ARGUMENT, "attention scratch: missing for %d columns", rows);
    // split_geom (attn_cols.rs:15-20): one run per 32 cache rows, at most 64 runs
    int splits = (n_ctx + 31) / 32;
    splits = splits < 1 ? 1 : (splits > 64 ? 64 : splits);
    return launch_decode_cols_f32(as_stream(stream), q, k_cache, v_cache, part_acc, part_ml, out,
                                  n_heads, n_kv, head_dim, n_ctx, pos0, rows, splits);
}

int hipml_set_decode_cta_slots(int slots) {
    if (slots < 0) return fail(HIPML_ERR_INVALID_ARGUMENT, "decode CTA slots %d", slots);
    g_cta_slots_override.store(slots);
    return 0;
}

int hipml_set_decode_body(int body) {
    if (body != 1 && body != 2)
        return fail(HIPML_ERR_INVALID_ARGUMENT, "decode body %d (1 values on mma.sync, 2 values on tcgen05)", body);
    decode_set_body(body);
    return 0;
}

int hipml_set_decode_fold_mode(int mode) {
    if (mode != 0 && mode != 1)
        return fail(HIPML_ERR_INVALID_ARGUMENT, "decode fold mode %d (0 inside the split pass, 1 own launch)", mode);
    decode_set_two_launch_fold(mode);
    return 0;
}

int hipml_decode_plan_quota(const int *lens, int slots, int splits, int n_kv, int cta_slots) {
    if (!lens || slots <= 0 || splits < 1 || n_kv <= 0 || cta_slots < 2 * slots * n_kv) return -1;
    return decode_plan_quota_host(lens, slots, splits, cta_slots, n_kv);
}

}  // extern "C"
