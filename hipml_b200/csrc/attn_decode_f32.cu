// Split-K decode over the f32 position-major cache for 1..R consecutive columns, and the
// matching multi-row append.
//
// CPU definition: crates/hipml-core/src/attention.rs:56-102 with seq = pos0 + c + 1 for
// column c. Kernels replaced: crates/hipml-kernels/kernels/attn_decode_cols_f32.hip:31-213
// (split pass + reduce) and kv_append_cols_f32.hip:11-31; launcher
// crates/hipml-kernels/src/attn_gpu/imp/attn_cols.rs:15-173. The key axis is cut into
// `splits` runs of `per = ceil(n_ctx / splits)` rows fixed in cache positions, so a column's
// arithmetic does not depend on how many columns share the launch. This is the `--kv f32`
// path of the reference: plain f32, one warp per (query head, run, column).
#include "params.cuh"

namespace hipml {

struct ColsParams {
    const float *q;        // [rows][n_heads*head_dim]
    const float *k;        // [n_ctx][n_kv*head_dim]
    const float *v;
    float *part_acc;       // [rows][n_heads][splits][head_dim]
    float *part_ml;        // [rows][n_heads][splits][2]
    int n_heads, n_kv, head_dim;
    int pos0, rows;
    float scale_log2;
    int splits, per;
};

namespace {

__global__ void __launch_bounds__(128) attn_decode_cols_f32(ColsParams p) {
    griddep_launch();
    griddep_wait();
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    const int col = blockIdx.y;
    if (warp >= p.n_heads * p.splits) return;
    const int h = warp / p.splits, split = warp - h * p.splits;
    const int kvh = h / (p.n_heads / p.n_kv);
    const int live = lane * 8 < p.head_dim;
    const int d0 = lane * 8;
    const int width = p.n_kv * p.head_dim;
    const int seq = p.pos0 + col + 1;
    const int lo = min(split * p.per, seq), hi = min(lo + p.per, seq);

    float qv[8];
    const float *q = p.q + ((size_t)col * p.n_heads + h) * p.head_dim;
#pragma unroll
    for (int j = 0; j < 8; j++) qv[j] = live ? q[d0 + j] * p.scale_log2 : 0.0f;
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    float m = -INFINITY, l = 0.0f;
    for (int pos = lo; pos < hi; pos++) {
        const size_t at = (size_t)pos * width + kvh * p.head_dim + d0;
        float part = 0.0f;
        if (live) {
#pragma unroll
            for (int j = 0; j < 8; j++) part += qv[j] * p.k[at + j];
        }
        const float s = warp_sum(part);
        const float m_new = fmaxf(m, s);
        const float corr = exp2f(m - m_new);
        const float w = exp2f(s - m_new);
        l = l * corr + w;
        m = m_new;
        if (live) {
#pragma unroll
            for (int j = 0; j < 8; j++) acc[j] = acc[j] * corr + w * p.v[at + j];
        }
    }
    const size_t slot = ((size_t)col * p.n_heads + h) * p.splits + split;
    if (live) {
#pragma unroll
        for (int j = 0; j < 8; j++) p.part_acc[slot * p.head_dim + d0 + j] = acc[j];
    }
    if (lane == 0) {
        p.part_ml[slot * 2] = m;
        p.part_ml[slot * 2 + 1] = l;
    }
}

}  // namespace

// Entry name, parameter list and linear launch shape of the reference's kernel: row c of k/v
// lands at cache row pos0 + c; threads [0,width) of a row copy K, [width,2*width) copy V.
extern "C" __global__ void kv_append_cols_f32(float *__restrict__ k_cache,
                                              float *__restrict__ v_cache,
                                              const float *__restrict__ k,
                                              const float *__restrict__ v, int pos0, int rows,
                                              int width) {
    griddep_launch();
    griddep_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= 2LL * width * rows) return;
    const int c = (int)(i / (2 * width));
    const int j = (int)(i - (long long)c * 2 * width);
    const size_t base = (size_t)(pos0 + c) * width;
    if (j < width)
        k_cache[base + j] = k[(size_t)c * width + j];
    else
        v_cache[base + j - width] = v[(size_t)c * width + j - width];
}

const void *lookup_cols_kernel(const char *name) {
    if (strcmp(name, "kv_append_cols_f32") == 0) return (const void *)kv_append_cols_f32;
    return nullptr;
}

int launch_decode_cols_f32(cudaStream_t stream, const float *q, const float *k, const float *v,
                           float *part_acc, float *part_ml, float *out, int n_heads, int n_kv,
                           int head_dim, int n_ctx, int pos0, int rows, int splits) {
    ColsParams p;
    p.q = q;
    p.k = k;
    p.v = v;
    p.part_acc = part_acc;
    p.part_ml = part_ml;
    p.n_heads = n_heads;
    p.n_kv = n_kv;
    p.head_dim = head_dim;
    p.pos0 = pos0;
    p.rows = rows;
    p.scale_log2 = (1.0f / sqrtf((float)head_dim)) * 1.4426950408889634f;
    p.splits = splits;
    p.per = (n_ctx + splits - 1) / splits;
    dim3 grid((n_heads * splits + 3) / 4, rows);
    if (int e = launch_pdl(attn_decode_cols_f32, grid, dim3(128), 0, stream, 1, p)) return e;
    if (int e = launch_status()) return e;
    return launch_decode_reduce(stream, part_acc, part_ml, out, n_heads, head_dim, splits, rows,
                                (long long)n_heads * splits * head_dim,
                                (long long)n_heads * splits * 2, (long long)n_heads * head_dim);
}

}  // namespace hipml
