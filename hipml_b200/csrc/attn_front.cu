// The attention front end and tail around the attention kernels: q|gate split, per-head RMS
// norm of q and k, M-RoPE of both, the output gate, and (fused form) the q8_0 append.
//
// CPU definition: crates/hipml-core/src/ops.rs:181-187 (rmsnorm), 260-309 (rope_multi),
// 315-329 (qg_split), 354-360 (q_gate), composed as in attention.rs:117-143. Kernels replaced:
// crates/hipml-kernels/kernels/attn_front_f32.hip:34-135, attn_chunk_f32.hip:22-98 and
// q_gate_f32.hip. The four kernels with the reference's names keep its parameter lists and
// launch shapes (a launch by name with the reference's argument array works unchanged) around
// bodies of this file's own; attn_front_rows_q8 is the form this library's own launchers use.
//
// attn_front_rows_q8: one CTA of 8 warps per token. The rotation angles depend on the
// position and the channel pair only, so the CTA computes the n_rot/2 (cos, sin) pairs once
// (f64 pow and sincos, as the definition does) and all heads share them. A warp owns a
// whole 256-wide head row: 8 values per lane (two 16-byte loads), the sum of squares by
// shuffles, the rotation partner (channel +- n_rot/2) in the lane n_rot/16 away. The K row
// leaves as a q8_0 cache row straight from the normalised, rotated registers and the V row
// is quantised beside it, so the chunk's split + norm + rope + append is one pass over the
// inputs: 108.7 KB per token at 24/4/256 (q|gate 48 KB in, q and gate 24 KB each out, k and v
// 8 KB in, 2.1 KB of cache rows out), HBM-bound.
#include "params.cuh"
#include "q8_pack.cuh"

namespace hipml {

namespace {

struct RopeSpec {
    int n_rot;
    int s0, s1, s2, s3;   // M-RoPE sections (all 0: every pair uses position id 0)
    float theta_base;
};

// Position id that feeds pair c (the section walk of the definition).
__device__ __forceinline__ int rope_pos(const RopeSpec &r, int c, const int (&pos)[4]) {
    const int sect = r.s0 + r.s1 + r.s2 + r.s3;
    if (sect <= 0) return pos[0];
    const int s = c % sect;
    if (s < r.s0) return pos[0];
    if (s < r.s0 + r.s1) return pos[1];
    if (s < r.s0 + r.s1 + r.s2) return pos[2];
    return pos[3];
}

__device__ __forceinline__ void rope_angle(const RopeSpec &r, int c, const int (&pos)[4], float &cs,
                                           float &sn) {
    const double freq = pow((double)r.theta_base, -2.0 * (double)c / (double)r.n_rot);
    const double ang = (double)rope_pos(r, c, pos) * freq;
    double s, co;
    sincos(ang, &s, &co);
    cs = (float)co;
    sn = (float)s;
}

constexpr int kMaxHeadDim = 256;

// Sum over the block (any block size that is a multiple of 32); `red` holds one float per warp.
__device__ __forceinline__ float block_sum(float v, float *red) {
    v = warp_sum(v);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = (blockDim.x + 31) >> 5;
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = 0.0f;
    for (int i = 0; i < nwarps; i++) t += red[i];
    __syncthreads();
    return t;
}

// One head row by one block, written from the CPU definition: y = x / sqrt(mean(x^2) + eps) * w
// (ops.rs:181-187), then the first n_rot channels rotated in NeoX pairs (c, c + n_rot / 2) by the
// angle position * theta^(-2c / n_rot) (ops.rs:260-309). No staging buffer: a thread owns whole
// pairs, reads both inputs, and writes both outputs, so `in` may be `out` (the K rows are
// rotated in place); channels past n_rot are only normalised.
__device__ __forceinline__ void head_row_norm_rope(const float *in, float *out, const float *weight,
                                                   int head_dim, const RopeSpec &rope,
                                                   const int (&pos)[4], float eps, float *red) {
    float sq = 0.0f;
    for (int d = threadIdx.x; d < head_dim; d += blockDim.x) sq = fmaf(in[d], in[d], sq);
    const float inv_rms = 1.0f / sqrtf(block_sum(sq, red) / (float)head_dim + eps);
    const int pairs = rope.n_rot >> 1;
    // work item i: a rotated pair for i < pairs, one plain channel after them
    for (int i = threadIdx.x; i < head_dim - pairs; i += blockDim.x) {
        if (i < pairs) {
            const float a = in[i] * inv_rms * weight[i];
            const float b = in[i + pairs] * inv_rms * weight[i + pairs];
            float cs, sn;
            rope_angle(rope, i, pos, cs, sn);
            out[i] = a * cs - b * sn;
            out[i + pairs] = a * sn + b * cs;
        } else {
            const int d = i + pairs;
            out[d] = in[d] * inv_rms * weight[d];
        }
    }
}

}  // namespace

// ---- entries by the reference's names --------------------------------------------------------
// Kept so that a launch by name with the reference's argument array and launch shape works
// unchanged (Kernel::launch, crates/hipml-hip/src/device.rs:543-580): the names, parameter
// lists and grids are the reference's (attn_front_f32.hip, attn_chunk_f32.hip), the bodies are
// this file's own (one routine for all three, written from the CPU definition above). The
// library's own launchers take the one-pass form further down instead.

// grid (n_heads + n_kv), block 256: blocks below n_heads take a query head (q half of its
// q|gate row -> q, gate half -> gate), the rest a key head (in place).
extern "C" __global__ void attn_front_f32(const float *__restrict__ qg, float *__restrict__ q,
                                          float *__restrict__ gate, float *k,
                                          const float *__restrict__ q_norm,
                                          const float *__restrict__ k_norm, int n_heads, int n_kv,
                                          int head_dim, int n_rot, int s0, int s1, int s2, int s3,
                                          const int *__restrict__ pos, float theta_base, float eps) {
    griddep_launch();
    griddep_wait();
    __shared__ float red[32];
    const int row = blockIdx.x;
    if (row >= n_heads + n_kv) return;
    const RopeSpec rope = {n_rot, s0, s1, s2, s3, theta_base};
    const int ids[4] = {pos[0], pos[1], pos[2], pos[3]};
    if (row < n_heads) {
        const float *pair = qg + (size_t)row * 2 * head_dim;
        for (int d = threadIdx.x; d < head_dim; d += blockDim.x)
            gate[(size_t)row * head_dim + d] = pair[head_dim + d];
        head_row_norm_rope(pair, q + (size_t)row * head_dim, q_norm, head_dim, rope, ids, eps, red);
    } else {
        float *key = k + (size_t)(row - n_heads) * head_dim;
        head_row_norm_rope(key, key, k_norm, head_dim, rope, ids, eps, red);
    }
}

// grid (n_heads, tokens), block head_dim: the q|gate rows of a chunk pulled apart.
extern "C" __global__ void qg_split_chunk_f32(const float *__restrict__ qg, float *__restrict__ q,
                                              float *__restrict__ gate, int n_heads, int head_dim,
                                              int tokens) {
    griddep_launch();
    griddep_wait();
    if ((int)blockIdx.y >= tokens || (int)blockIdx.x >= n_heads) return;
    const size_t row = (size_t)blockIdx.y * n_heads + blockIdx.x;
    // element e of the joint row goes to q (first half) or gate (second half)
    for (int e = threadIdx.x; e < 2 * head_dim; e += blockDim.x) {
        const float x = qg[row * 2 * head_dim + e];
        if (e < head_dim)
            q[row * head_dim + e] = x;
        else
            gate[row * head_dim + e - head_dim] = x;
    }
}

// grid (n_heads + n_kv, tokens), block head_dim: norm + rope of a chunk's rows in place; token t
// sits at text position pos0 + t (all four position ids equal).
extern "C" __global__ void norm_rope_chunk_f32(float *__restrict__ q, float *__restrict__ k,
                                               const float *__restrict__ qw,
                                               const float *__restrict__ kw, int n_heads, int n_kv,
                                               int head_dim, int n_rot, float theta_base, float eps,
                                               int pos0, int tokens) {
    griddep_launch();
    griddep_wait();
    __shared__ float red[32];
    const int t = blockIdx.y, row = blockIdx.x;
    if (t >= tokens || row >= n_heads + n_kv) return;
    const RopeSpec rope = {n_rot, 0, 0, 0, 0, theta_base};
    const int ids[4] = {pos0 + t, pos0 + t, pos0 + t, pos0 + t};
    float *x = row < n_heads ? q + ((size_t)t * n_heads + row) * head_dim
                             : k + ((size_t)t * n_kv + (row - n_heads)) * head_dim;
    head_row_norm_rope(x, x, row < n_heads ? qw : kw, head_dim, rope, ids, eps, red);
}

// y[i] = q[i] * sigmoid(gate[i]); one thread per element.
extern "C" __global__ void q_gate_f32(const float *__restrict__ q, const float *__restrict__ gate,
                                      float *__restrict__ y, int n) {
    griddep_launch();
    griddep_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) y[i] = q[i] * (1.0f / (1.0f + expf(-gate[i])));
}

// ---- this library's forms --------------------------------------------------------------------

namespace {

// 16 bytes per thread, grid-stride.
__global__ void __launch_bounds__(256) q_gate_v4(const float4 *__restrict__ q,
                                                 const float4 *__restrict__ gate,
                                                 float4 *__restrict__ y, size_t n4) {
    griddep_launch();
    griddep_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4;
         i += (size_t)gridDim.x * blockDim.x) {
        const float4 a = q[i], g = gate[i];
        y[i] = make_float4(a.x * (1.0f / (1.0f + expf(-g.x))), a.y * (1.0f / (1.0f + expf(-g.y))),
                           a.z * (1.0f / (1.0f + expf(-g.z))), a.w * (1.0f / (1.0f + expf(-g.w))));
    }
}

struct FrontRowsParams {
    const float *qg;      // [tokens][n_heads][512]
    const float *k;       // [tokens][n_kv][256]
    const float *v;       // [tokens][n_kv][256]
    float *q;             // [tokens][n_heads][256]
    float *gate;          // [tokens][n_heads][256]
    float *k_out;         // optional: the normalised, rotated k rows as f32
    const float *q_norm, *k_norm;
    unsigned char *kc, *vc;   // optional q8_0 caches (head-major, `stride` rows per head)
    const int *pos4;      // optional device [4]: M-RoPE position ids of the (single) token
    const int *step;      // optional device: step[0] = cache row of the (single) token
    int n_heads, n_kv, stride, pos0, tokens;
    RopeSpec rope;
    float eps;
};

__device__ __forceinline__ void load8(const float *p, float (&x)[8]) {
    const float4 a = __ldg(reinterpret_cast<const float4 *>(p));
    const float4 b = __ldg(reinterpret_cast<const float4 *>(p) + 1);
    x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w;
    x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
}
__device__ __forceinline__ void store8(float *p, const float (&x)[8]) {
    reinterpret_cast<float4 *>(p)[0] = make_float4(x[0], x[1], x[2], x[3]);
    reinterpret_cast<float4 *>(p)[1] = make_float4(x[4], x[5], x[6], x[7]);
}

// RMS norm + rope of the 256-wide row held 8 values per lane (values 8*lane .. 8*lane+7).
__device__ __forceinline__ void norm_rope_lane8(float (&x)[8], const float *w, int lane, int n_rot,
                                                float eps, const float *cs, const float *sn) {
    float acc = 0.0f;
#pragma unroll
    for (int j = 0; j < 8; j++) acc = fmaf(x[j], x[j], acc);
    const float scale = 1.0f / sqrtf(warp_sum(acc) / 256.0f + eps);
    float wv[8];
    load8(w + 8 * lane, wv);
#pragma unroll
    for (int j = 0; j < 8; j++) x[j] = x[j] * scale * wv[j];
    // the partner of channel c < half is c + half: same j, lane + half/8 (and back)
    const int half = n_rot >> 1, hop = half >> 3;
    const bool low = 8 * lane < half, rot = 8 * lane < n_rot;
#pragma unroll
    for (int j = 0; j < 8; j++) {
        const float other = __shfl_sync(0xffffffffu, x[j], (low ? lane + hop : lane - hop) & 31);
        if (rot) {
            const int c = (low ? 8 * lane : 8 * lane - half) + j;
            x[j] = low ? x[j] * cs[c] - other * sn[c] : other * sn[c] + x[j] * cs[c];
        }
    }
}

// grid (tokens), block 256.
__global__ void __launch_bounds__(256) attn_front_rows_q8(FrontRowsParams p) {
    __shared__ float cs[kMaxHeadDim / 2], sn[kMaxHeadDim / 2];
    __shared__ __align__(16) unsigned char img[8][kMaxRowBytes];
    griddep_launch();
    griddep_wait();   // positions and rows may come from a grid that is still running
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int p4[4];
    if (p.pos4) {
        p4[0] = p.pos4[0]; p4[1] = p.pos4[1]; p4[2] = p.pos4[2]; p4[3] = p.pos4[3];
    } else {
        p4[0] = p4[1] = p4[2] = p4[3] = p.pos0 + t;
    }
    const int half = p.rope.n_rot >> 1;
    for (int c = threadIdx.x; c < half; c += blockDim.x) rope_angle(p.rope, c, p4, cs[c], sn[c]);
    __syncthreads();
    const int cache_row = p.step ? p.step[0] : p.pos0 + t;
    const int rows = p.n_heads + 2 * p.n_kv;
    for (int r = warp; r < rows; r += 8) {
        float x[8];
        if (r < p.n_heads) {
            const float *src = p.qg + ((size_t)t * p.n_heads + r) * 512;
            float g[8];
            load8(src + 8 * lane, x);
            load8(src + 256 + 8 * lane, g);
            store8(p.gate + ((size_t)t * p.n_heads + r) * 256 + 8 * lane, g);
            norm_rope_lane8(x, p.q_norm, lane, p.rope.n_rot, p.eps, cs, sn);
            store8(p.q + ((size_t)t * p.n_heads + r) * 256 + 8 * lane, x);
            continue;
        }
        const bool is_k = r < p.n_heads + p.n_kv;
        const int h = is_k ? r - p.n_heads : r - p.n_heads - p.n_kv;
        load8((is_k ? p.k : p.v) + ((size_t)t * p.n_kv + h) * 256 + 8 * lane, x);
        if (is_k) {
            norm_rope_lane8(x, p.k_norm, lane, p.rope.n_rot, p.eps, cs, sn);
            if (p.k_out) store8(p.k_out + ((size_t)t * p.n_kv + h) * 256 + 8 * lane, x);
        }
        unsigned char *cache = is_k ? p.kc : p.vc;
        if (cache) {
            q8_put8(make_float4(x[0], x[1], x[2], x[3]), make_float4(x[4], x[5], x[6], x[7]), lane,
                    img[warp]);
            __syncwarp();
            row_store(cache + q8_row_offset(h, p.stride, cache_row, 256), img[warp], kMaxRowBytes, lane,
                      32);
            __syncwarp();
        }
    }
}

}  // namespace

const void *lookup_front_kernel(const char *name) {
    if (strcmp(name, "attn_front_f32") == 0) return (const void *)attn_front_f32;
    if (strcmp(name, "qg_split_chunk_f32") == 0) return (const void *)qg_split_chunk_f32;
    if (strcmp(name, "norm_rope_chunk_f32") == 0) return (const void *)norm_rope_chunk_f32;
    if (strcmp(name, "q_gate_f32") == 0) return (const void *)q_gate_f32;
    return nullptr;
}

int launch_q_gate(cudaStream_t stream, const float *q, const float *gate, float *y, long long n) {
    if (n <= 0) return 0;
    const size_t align = reinterpret_cast<size_t>(q) | reinterpret_cast<size_t>(gate) |
                         reinterpret_cast<size_t>(y);
    if (n % 4 == 0 && (align & 15) == 0) {
        const size_t n4 = (size_t)n / 4;
        size_t blocks = (n4 + 255) / 256;
        if (blocks > 148 * 16) blocks = 148 * 16;
        return launch_pdl(q_gate_v4, dim3((unsigned)blocks), dim3(256), 0, stream, 1,
                          reinterpret_cast<const float4 *>(q), reinterpret_cast<const float4 *>(gate),
                          reinterpret_cast<float4 *>(y), n4);
    }
    if (n > 0x7fffffffLL) return fail(HIPML_ERR_INVALID_ARGUMENT, "q_gate: %lld elements", n);
    return launch_pdl(q_gate_f32, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, 1, q, gate, y,
                      (int)n);
}

int launch_front_rows_q8(cudaStream_t stream, const float *qg, const float *k, const float *v,
                         float *q, float *gate, float *k_out, const float *q_norm,
                         const float *k_norm, void *k_cache, void *v_cache, int n_heads, int n_kv,
                         int n_rot, const int *sections, const int *pos4, const int *step, int pos0,
                         int tokens, int stride, float theta_base, float eps) {
    FrontRowsParams p;
    p.qg = qg;
    p.k = k;
    p.v = v;
    p.q = q;
    p.gate = gate;
    p.k_out = k_out;
    p.q_norm = q_norm;
    p.k_norm = k_norm;
    p.kc = reinterpret_cast<unsigned char *>(k_cache);
    p.vc = reinterpret_cast<unsigned char *>(v_cache);
    p.pos4 = pos4;
    p.step = step;
    p.n_heads = n_heads;
    p.n_kv = n_kv;
    p.stride = stride;
    p.pos0 = pos0;
    p.tokens = tokens;
    p.rope.n_rot = n_rot;
    p.rope.s0 = sections ? sections[0] : 0;
    p.rope.s1 = sections ? sections[1] : 0;
    p.rope.s2 = sections ? sections[2] : 0;
    p.rope.s3 = sections ? sections[3] : 0;
    p.rope.theta_base = theta_base;
    p.eps = eps;
    return launch_pdl(attn_front_rows_q8, dim3(tokens), dim3(256), 0, stream, 1, p);
}

}  // namespace hipml
