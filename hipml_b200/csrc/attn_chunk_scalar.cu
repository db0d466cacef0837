// Causal chunk (prefill) attention, scalar f32 body, and the split combine.
//
// CPU definition: crates/hipml-core/src/attention.rs:56-102 called per query row with
// seq = pos0 + t + 1 (crates/hipml-cli/src/attn_chunk_parity.rs:44-58). This body is the
// A/B and cross-check kernel (the role crates/hipml-kernels/kernels/attn_chunk_f32.hip
// plays in the reference): one warp per (query row, query head), online softmax in log2
// units, every operand in f32. It reads either cache format directly, needs no workspace
// and accepts any head_dim in 32..256 step 32; the tensor-core kernel is the fast path.
//
// attn_chunk_combine_f32 replaces crates/hipml-kernels/kernels/attn_chunk_split.hip:343-376
// and keeps its name, parameter list and launch shape.
#include "params.cuh"
#include "q8_pack.cuh"

namespace hipml {


namespace {

__global__ void __launch_bounds__(128) attn_chunk_scalar(ChunkScalarParams p) {
    griddep_launch();
    griddep_wait();
    const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    const int nsp = p.splits < 2 ? 1 : p.splits;
    const long long total = (long long)p.tokens * p.n_heads * nsp;
    if (warp >= total) return;
    const int sp = (int)(warp % nsp);
    const long long th = warp / nsp;
    const int h = (int)(th % p.n_heads);
    const int t = (int)(th / p.n_heads);
    const int group = p.n_heads / p.n_kv;
    const int kvh = h / group;
    const int nb = p.head_dim >> 5;
    const int blk = lane >> 2, sub = lane & 3;
    const bool live = blk < nb;
    const int d0 = blk * kBlock + sub * 8;
    const int width = p.n_kv * p.head_dim;

    // Row t sees cache rows 0..pos0+t; slice sp of that range when split.
    const long long bound = (long long)p.pos0 + t + 1;
    const int lo = (int)(bound * sp / nsp);
    const int hi = (int)(bound * (sp + 1) / nsp);

    float qv[8];
    const float *q = p.q + ((size_t)t * p.n_heads + h) * p.head_dim;
#pragma unroll
    for (int j = 0; j < 8; j++) qv[j] = live ? q[d0 + j] * p.scale_log2 : 0.0f;

    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    float m = -INFINITY, l = 0.0f;
    for (int pos = lo; pos < hi; pos++) {
        float kx[8], vx[8];
        if (live) {
            if (p.kv_dtype == 0) {
                const float *kr = (const float *)p.k + (size_t)pos * width + kvh * p.head_dim + d0;
                const float *vr = (const float *)p.v + (size_t)pos * width + kvh * p.head_dim + d0;
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    kx[j] = kr[j];
                    vx[j] = vr[j];
                }
            } else if (p.kv_dtype == 2) {
                // q4_0: this lane's dims are the low (sub < 2) or high nibbles of 8 bytes
                const size_t row = q4_row_offset(kvh, p.stride, pos, p.head_dim) +
                                   (size_t)blk * kQ4BlockBytes;
                const unsigned char *kb = (const unsigned char *)p.k + row;
                const unsigned char *vb = (const unsigned char *)p.v + row;
                const float dk = half_bits_to_float(*(const unsigned short *)kb);
                const float dv = half_bits_to_float(*(const unsigned short *)vb);
                const unsigned short *kc = (const unsigned short *)(kb + 2 + (sub & 1) * 8);
                const unsigned short *vc = (const unsigned short *)(vb + 2 + (sub & 1) * 8);
                const int shift = (sub >> 1) * 4;
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const unsigned short a = kc[j], b = vc[j];
                    kx[2 * j] = dk * ((float)((a >> shift) & 0xf) - 8.0f);
                    kx[2 * j + 1] = dk * ((float)((a >> (8 + shift)) & 0xf) - 8.0f);
                    vx[2 * j] = dv * ((float)((b >> shift) & 0xf) - 8.0f);
                    vx[2 * j + 1] = dv * ((float)((b >> (8 + shift)) & 0xf) - 8.0f);
                }
            } else {
                const size_t row = q8_row_offset(kvh, p.stride, pos, p.head_dim) +
                                   (size_t)blk * kQ8BlockBytes;
                const unsigned char *kb = (const unsigned char *)p.k + row;
                const unsigned char *vb = (const unsigned char *)p.v + row;
                const float dk = half_bits_to_float(*(const unsigned short *)kb);
                const float dv = half_bits_to_float(*(const unsigned short *)vb);
                const unsigned short *kc = (const unsigned short *)(kb + 2 + sub * 8);
                const unsigned short *vc = (const unsigned short *)(vb + 2 + sub * 8);
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const unsigned short a = kc[j], b = vc[j];
                    kx[2 * j] = dk * (float)(signed char)(a & 0xff);
                    kx[2 * j + 1] = dk * (float)(signed char)(a >> 8);
                    vx[2 * j] = dv * (float)(signed char)(b & 0xff);
                    vx[2 * j + 1] = dv * (float)(signed char)(b >> 8);
                }
            }
        }
        float part = 0.0f;
        if (live) {
#pragma unroll
            for (int j = 0; j < 8; j++) part += qv[j] * kx[j];
        }
        const float s = warp_sum(part);
        const float m_new = fmaxf(m, s);
        const float corr = exp2f(m - m_new);
        const float w = exp2f(s - m_new);
        l = l * corr + w;
        m = m_new;
        if (live) {
#pragma unroll
            for (int j = 0; j < 8; j++) acc[j] = acc[j] * corr + w * vx[j];
        }
    }
    if (p.splits < 2) {
        if (live) {
            float *o = p.out + ((size_t)t * p.n_heads + h) * p.head_dim + d0;
            const float inv = l > 0.0f ? 1.0f / l : 0.0f;
#pragma unroll
            for (int j = 0; j < 8; j++) o[j] = acc[j] * inv;
        }
    } else {
        const size_t slot = ((size_t)sp * p.qslots + t) * p.n_heads + h;
        if (live) {
            float *o = p.part_acc + slot * p.head_dim + d0;
#pragma unroll
            for (int j = 0; j < 8; j++) o[j] = acc[j];
        }
        if (lane == 0) {
            p.part_ml[slot * 2] = m;
            p.part_ml[slot * 2 + 1] = l;
        }
    }
}

}  // namespace

// grid (qslots, n_heads), block head_dim: out[t][h][:] = sum_s acc_s*2^(m_s-M) / sum_s l_s*2^(m_s-M).
// Rows >= tokens are scratch padding and are skipped. An empty slice carries sum 0 and
// any max (-inf here, -1e30 in the reference's split kernels); both weigh in as 0.
extern "C" __global__ void attn_chunk_combine_f32(const float *__restrict__ part_acc,
                                                  const float *__restrict__ part_ml,
                                                  float *__restrict__ out, int n_heads,
                                                  int head_dim, int tokens, int qslots,
                                                  int splits) {
    griddep_launch();
    griddep_wait();
    const int t = blockIdx.x, h = blockIdx.y, d = threadIdx.x;
    if (t >= tokens || d >= head_dim) return;
    float big = -INFINITY;
    for (int s = 0; s < splits; s++) {
        const size_t slot = ((size_t)s * qslots + t) * n_heads + h;
        if (part_ml[slot * 2 + 1] > 0.0f) big = fmaxf(big, part_ml[slot * 2]);
    }
    float num = 0.0f, den = 0.0f;
    for (int s = 0; s < splits; s++) {
        const size_t slot = ((size_t)s * qslots + t) * n_heads + h;
        const float l = part_ml[slot * 2 + 1];
        if (!(l > 0.0f)) continue;
        const float w = exp2f(part_ml[slot * 2] - big);
        num += part_acc[slot * head_dim + d] * w;
        den += l * w;
    }
    out[((size_t)t * n_heads + h) * head_dim + d] = den > 0.0f ? num / den : 0.0f;
}

int launch_chunk_scalar(cudaStream_t stream, const ChunkScalarParams &p) {
    const int nsp = p.splits < 2 ? 1 : p.splits;
    const long long warps = (long long)p.tokens * p.n_heads * nsp;
    if (warps == 0) return 0;
    const long long blocks = (warps + 3) / 4;
    return launch_pdl(attn_chunk_scalar, dim3((unsigned)blocks), dim3(128), 0, stream, 1, p);
}

// The same fold for head_dim 256 with 16-byte accesses: 64 threads per (row, head), four
// (row, head) pairs per CTA. What launch_chunk_combine uses when the shape allows; the kernel
// above keeps the reference's launch shape for launches by name.
__global__ void __launch_bounds__(256) attn_chunk_combine_256(const float *__restrict__ part_acc,
                                                              const float *__restrict__ part_ml,
                                                              float *__restrict__ out, int n_heads,
                                                              int tokens, int qslots, int splits,
                                                              const float *__restrict__ gate) {
    griddep_launch();
    griddep_wait();
    const long long pair = (long long)blockIdx.x * 4 + (threadIdx.x >> 6);
    if (pair >= (long long)tokens * n_heads) return;
    const int t = (int)(pair / n_heads), h = (int)(pair - (long long)t * n_heads);
    const int d4 = threadIdx.x & 63;
    float big = -INFINITY;
    for (int s = 0; s < splits; s++) {
        const float2 ml = *reinterpret_cast<const float2 *>(
            part_ml + (((size_t)s * qslots + t) * n_heads + h) * 2);
        if (ml.y > 0.0f) big = fmaxf(big, ml.x);
    }
    float4 num = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    float den = 0.0f;
    for (int s = 0; s < splits; s++) {
        const size_t slot = ((size_t)s * qslots + t) * n_heads + h;
        const float2 ml = *reinterpret_cast<const float2 *>(part_ml + slot * 2);
        if (!(ml.y > 0.0f)) continue;
        const float w = exp2f(ml.x - big);
        const float4 a = __ldg(reinterpret_cast<const float4 *>(part_acc + slot * 256) + d4);
        num.x += a.x * w; num.y += a.y * w; num.z += a.z * w; num.w += a.w * w;
        den += ml.y * w;
    }
    const bool ok = den > 0.0f;
    float4 o = make_float4(ok ? num.x / den : 0.0f, ok ? num.y / den : 0.0f,
                           ok ? num.z / den : 0.0f, ok ? num.w / den : 0.0f);
    if (gate) {
        const float4 g = reinterpret_cast<const float4 *>(gate + ((size_t)t * n_heads + h) * 256)[d4];
        o.x *= 1.0f / (1.0f + expf(-g.x));
        o.y *= 1.0f / (1.0f + expf(-g.y));
        o.z *= 1.0f / (1.0f + expf(-g.z));
        o.w *= 1.0f / (1.0f + expf(-g.w));
    }
    reinterpret_cast<float4 *>(out + ((size_t)t * n_heads + h) * 256)[d4] = o;
}

int launch_chunk_combine(cudaStream_t stream, const float *part_acc, const float *part_ml,
                         float *out, int n_heads, int head_dim, int tokens, int qslots,
                         int splits, const float *gate) {
    if (head_dim == 256 &&
        ((reinterpret_cast<size_t>(part_acc) | reinterpret_cast<size_t>(out)) & 15) == 0 &&
        (reinterpret_cast<size_t>(part_ml) & 7) == 0) {
        const long long pairs = (long long)tokens * n_heads;
        return launch_pdl(attn_chunk_combine_256, dim3((unsigned)((pairs + 3) / 4)), dim3(256), 0, stream, 1,
                          part_acc, part_ml, out, n_heads, tokens, qslots, splits, gate);
    }
    if (gate) return fail(HIPML_ERR_INVALID_ARGUMENT, "gated combine: head_dim 256, 16-byte aligned rows");
    dim3 grid(qslots, n_heads);
    return launch_pdl(attn_chunk_combine_f32, grid, dim3(head_dim), 0, stream, 1, part_acc, part_ml, out,
                      n_heads, head_dim, tokens, qslots, splits);
}

const void *lookup_chunk_kernel(const char *name) {
    if (strcmp(name, "attn_chunk_combine_f32") == 0) return (const void *)attn_chunk_combine_f32;
    return nullptr;
}

}  // namespace hipml
