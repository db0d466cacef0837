// Split-K flash-decode over the q8_0 KV cache: one query token per sequence
// (or per slot), GQA, partial (acc, max, sum) triples per key split, and the
// reduce that folds them.
//
// CPU definition: crates/hipml-core/src/ops.rs:449-518 (attn_decode_kv).
// Kernels replaced: crates/hipml-kernels/kernels/attn_decode_kv_w.hip:92-285
// (single stream), attn_decode_kv.hip:251-374,427-484 (multi-slot) and
// attn_decode_kv.hip:491-532 (reduce). Partial layout (shared with the
// reference): part_acc[(h*splits + s)*D + d], part_ml[(h*splits + s)*2 + {0: max in
// log2 units, 1: sum}]; slot b adds b*acc_slot / b*ml_slot.
//
// Two bodies:
//  * attn_decode_kv_tc  -- head_dim 256. A CTA owns one (KV head, split[, slot]) and
//    streams its rows through a double-buffered shared-memory ring with 16-byte
//    asynchronous copies (rows are 272 B, 16-byte aligned, and consecutive positions
//    of one head are contiguous, so a tile is one linear run). Both contractions run
//    on the tensor cores with f16 operands built in registers: int8 codes are exact
//    in f16, the query and the softmax weights are split into f16 high + low parts
//    stacked along the M dimension of one m16n8k16 tile (rows 0..7 high, 8..15 low),
//    and the per-block f16 scales are applied in f32 (K side: on the 32-wide partial
//    dot products; V side: folded into the weight operand), so results agree with the
//    f32 definition to ~1e-6. This keeps the CUDA cores for byte unpacking only: at
//    12 f32 FMA per cache byte a scalar kernel cannot keep up with HBM3e.
//  * attn_decode_kv_scalar -- any head_dim in 32..256 step 32, one warp per
//    (query head, split), plain f32. Kept as the A/B kernel (selector 6).
#include "params.cuh"

namespace hipml {


namespace {

__device__ __forceinline__ void split_range(const DecodeParams &p, int slot, int split, int &lo,
                                            int &hi) {
    const int len = p.len[slot * p.len_stride + p.len_offset];
    const int span = p.by_stride ? p.stride : len;
    const int per = (span + p.splits - 1) / p.splits;
    lo = min(split * per, len);
    hi = min(lo + per, len);
    if (split * per >= len) hi = lo;
}

// ------------------------------------------------------------ scalar body

__global__ void __launch_bounds__(128) attn_decode_kv_scalar(DecodeParams p) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    const int slot = blockIdx.y;
    if (warp >= p.n_heads * p.splits) return;
    const int h = warp / p.splits, split = warp - h * p.splits;
    const int group = p.n_heads / p.n_kv;
    const int kvh = h / group;
    const int nb = p.head_dim >> 5;
    const int blk = lane >> 2, sub = lane & 3;
    const bool live = blk < nb;
    const int d0 = blk * kBlock + sub * 8;

    int lo, hi;
    split_range(p, slot, split, lo, hi);

    float qv[8];
    const float *q = p.q + (size_t)slot * p.q_slot + (size_t)h * p.head_dim;
#pragma unroll
    for (int j = 0; j < 8; j++) qv[j] = live ? q[d0 + j] * p.scale_log2 : 0.0f;

    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    float m = -INFINITY, l = 0.0f;
    const size_t head_off = (size_t)slot * p.kv_slot_bytes;
    for (int pos = lo; pos < hi; pos++) {
        const size_t row = head_off + q8_row_offset(kvh, p.stride, pos, p.head_dim) +
                           (size_t)blk * kQ8BlockBytes;
        float part = 0.0f;
        if (live) {
            const unsigned char *kb = p.k + row;
            const float d = half_bits_to_float(*reinterpret_cast<const unsigned short *>(kb));
            const unsigned short *c = reinterpret_cast<const unsigned short *>(kb + 2 + sub * 8);
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const unsigned short w = c[j];
                part += qv[2 * j] * (d * (float)(signed char)(w & 0xff));
                part += qv[2 * j + 1] * (d * (float)(signed char)(w >> 8));
            }
        }
        const float s = warp_sum(part);
        const float m_new = fmaxf(m, s);
        const float corr = exp2f(m - m_new);
        const float w = exp2f(s - m_new);
        l = l * corr + w;
        m = m_new;
        if (live) {
            const unsigned char *vb = p.v + row;
            const float d = half_bits_to_float(*reinterpret_cast<const unsigned short *>(vb));
            const unsigned short *c = reinterpret_cast<const unsigned short *>(vb + 2 + sub * 8);
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const unsigned short cw = c[j];
                acc[2 * j] = acc[2 * j] * corr + w * (d * (float)(signed char)(cw & 0xff));
                acc[2 * j + 1] = acc[2 * j + 1] * corr + w * (d * (float)(signed char)(cw >> 8));
            }
        }
    }
    float *pa = p.part_acc + (size_t)slot * p.acc_slot +
                ((size_t)h * p.splits + split) * p.head_dim;
    if (live) {
#pragma unroll
        for (int j = 0; j < 8; j++) pa[d0 + j] = acc[j];
    }
    if (lane == 0) {
        float *pm = p.part_ml + (size_t)slot * p.ml_slot + ((size_t)h * p.splits + split) * 2;
        pm[0] = m;
        pm[1] = l;
    }
}

// -------------------------------------------------------- tensor-core body

constexpr int kTcTile = 64;                        // keys per shared-memory tile
constexpr int kTcRowBytes = 8 * kQ8BlockBytes;     // 272
constexpr int kTcTileBytes = kTcTile * kTcRowBytes;
constexpr int kTcThreads = 128;
constexpr float kPScale = 1024.0f;                 // keeps p*scale in f16's normal range

// Dynamic shared memory: K[2] | V[2] tiles, then the query and the score tile.
constexpr int kTcSmemBytes = 4 * kTcTileBytes + 8 * 256 * 4 + 8 * kTcTile * 4;

__device__ __forceinline__ void cp_async_16(void *smem, const void *gmem) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

__device__ __forceinline__ void mma_16816(float (&c)[4], const unsigned (&a)[4], unsigned b0,
                                          unsigned b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// The eight "logical words" of a block: four codes each, 4-byte aligned in the row.
// Odd blocks start 2 bytes past a word boundary, so their codes are aligned:
// word j holds codes 4j..4j+3. Even blocks start on a word boundary, so the scale
// shares a word with codes 0,1: words 0..6 hold codes 4j+2..4j+5 and word 7 is
// stitched from codes 0,1 and 30,31. Element order inside the contraction is
// free as long as both operands use the same one.
__device__ __forceinline__ unsigned block_word(const unsigned *row, int blk, int j) {
    const int m = blk >> 1;
    if (blk & 1) return row[17 * m + 9 + j];
    if (j < 7) return row[17 * m + 1 + j];
    return __byte_perm(row[17 * m], row[17 * m + 8], 0x5432);
}

// head_dim index of byte i of logical word j of block blk.
__device__ __forceinline__ int block_word_dim(int blk, int j, int i) {
    if (blk & 1) return blk * 32 + 4 * j + i;
    if (j < 7) return blk * 32 + 4 * j + 2 + i;
    return blk * 32 + (i < 2 ? i : 28 + i);
}

__device__ __forceinline__ float block_scale(const unsigned char *row, int blk) {
    return half_bits_to_float(*reinterpret_cast<const unsigned short *>(row + blk * kQ8BlockBytes));
}

// Two int8 codes (bytes lo_sel of x) as an exact half2: 0x64xx is 1024 + xx, and x was
// biased by 128, so subtracting 1152 gives the signed code.
__device__ __forceinline__ unsigned codes_to_half2(unsigned biased, unsigned selector) {
    const unsigned h = __byte_perm(biased, 0x64646464u, selector);
    const __half2 r = __hsub2(*reinterpret_cast<const __half2 *>(&h), __half2half2(__ushort_as_half(0x6480)));
    return *reinterpret_cast<const unsigned *>(&r);
}

__device__ __forceinline__ unsigned pack_half2(__half lo, __half hi) {
    const __half2 r = __halves2half2(lo, hi);
    return *reinterpret_cast<const unsigned *>(&r);
}

__global__ void __launch_bounds__(kTcThreads) attn_decode_kv_tc(DecodeParams p) {
    extern __shared__ __align__(16) unsigned char smem[];
    unsigned char *ktile[2] = {smem, smem + kTcTileBytes};
    unsigned char *vtile[2] = {smem + 2 * kTcTileBytes, smem + 3 * kTcTileBytes};
    float *qs = reinterpret_cast<float *>(smem + 4 * kTcTileBytes);  // [8][256], pre-scaled
    float *ss = qs + 8 * 256;                                        // [8][kTcTile] scores

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int slot = blockIdx.y;
    const int kvh = blockIdx.x / p.splits, split = blockIdx.x - kvh * p.splits;
    const int group = p.n_heads / p.n_kv;

    int lo, hi;
    split_range(p, slot, split, lo, hi);

    // Query rows of this KV head's group, scaled into log2 units; absent rows are zero.
    const float *q = p.q + (size_t)slot * p.q_slot + (size_t)kvh * group * 256;
    for (int i = tid; i < 8 * 256; i += kTcThreads)
        qs[i] = (i >> 8) < group ? q[i] * p.scale_log2 : 0.0f;

    const size_t head_byte = (size_t)slot * p.kv_slot_bytes + q8_row_offset(kvh, p.stride, 0, 256);
    const unsigned char *kbase = p.k + head_byte;
    const unsigned char *vbase = p.v + head_byte;

    auto prefetch = [&](int tile, int buf) {
        const int r0 = lo + tile * kTcTile;
        const int nrows = min(kTcTile, hi - r0);
        if (nrows > 0) {
            const size_t off = (size_t)r0 * kTcRowBytes;
            const int chunks = nrows * (kTcRowBytes / 16);
            for (int i = tid; i < chunks; i += kTcThreads) {
                cp_async_16(ktile[buf] + i * 16, kbase + off + (size_t)i * 16);
                cp_async_16(vtile[buf] + i * 16, vbase + off + (size_t)i * 16);
            }
        }
        cp_async_commit();
    };

    const int ntiles = (hi - lo + kTcTile - 1) / kTcTile;
    if (ntiles > 0) prefetch(0, 0);
    __syncthreads();  // qs visible

    // A fragments of the query for all 16 k-steps: rows 0..7 = f16 high part of head g,
    // rows 8..15 = f16 low part, contraction slots in block_word order.
    unsigned qa[16][4];
#pragma unroll
    for (int ks = 0; ks < 16; ks++) {
        const int blk = ks >> 1, j = (ks & 1) * 4 + t;
        float x[4];
#pragma unroll
        for (int i = 0; i < 4; i++) x[i] = qs[g * 256 + block_word_dim(blk, j, i)];
        __half xh[4], xl[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            xh[i] = __float2half_rn(x[i]);
            xl[i] = __float2half_rn(x[i] - __half2float(xh[i]));
        }
        qa[ks][0] = pack_half2(xh[0], xh[1]);
        qa[ks][1] = pack_half2(xl[0], xl[1]);
        qa[ks][2] = pack_half2(xh[2], xh[3]);
        qa[ks][3] = pack_half2(xl[2], xl[3]);
    }

    float acc[2][4][4];  // [block of this warp][byte i][c0..c3]
#pragma unroll
    for (int a = 0; a < 2; a++)
#pragma unroll
        for (int i = 0; i < 4; i++)
#pragma unroll
            for (int c = 0; c < 4; c++) acc[a][i][c] = 0.0f;
    float m_run = -INFINITY, l_run = 0.0f;

    for (int tile = 0; tile < ntiles; tile++) {
        const int buf = tile & 1;
        if (tile + 1 < ntiles) {
            prefetch(tile + 1, buf ^ 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const int r0 = lo + tile * kTcTile;
        const int nvalid = min(kTcTile, hi - r0);

        // ---- scores: warp w owns keys [16w, 16w+16) of the tile, all 256 dims.
        {
            float s[2][2] = {{0.0f, 0.0f}, {0.0f, 0.0f}};
#pragma unroll
            for (int blk = 0; blk < 8; blk++) {
                float c[2][4] = {{0, 0, 0, 0}, {0, 0, 0, 0}};
#pragma unroll
                for (int kk = 0; kk < 2; kk++) {
#pragma unroll
                    for (int nt = 0; nt < 2; nt++) {
                        const int key = warp * 16 + nt * 8 + g;
                        const unsigned *row =
                            reinterpret_cast<const unsigned *>(ktile[buf] + key * kTcRowBytes);
                        const unsigned w = block_word(row, blk, kk * 4 + t) ^ 0x80808080u;
                        mma_16816(c[nt], qa[blk * 2 + kk], codes_to_half2(w, 0x4140),
                                  codes_to_half2(w, 0x4342));
                    }
                }
#pragma unroll
                for (int nt = 0; nt < 2; nt++) {
                    const int key = warp * 16 + nt * 8 + 2 * t;
                    const float d0 = block_scale(ktile[buf] + key * kTcRowBytes, blk);
                    const float d1 = block_scale(ktile[buf] + (key + 1) * kTcRowBytes, blk);
                    s[nt][0] += d0 * (c[nt][0] + c[nt][2]);
                    s[nt][1] += d1 * (c[nt][1] + c[nt][3]);
                }
            }
#pragma unroll
            for (int nt = 0; nt < 2; nt++) {
                const int key = warp * 16 + nt * 8 + 2 * t;
                ss[g * kTcTile + key] = key < nvalid ? s[nt][0] : -INFINITY;
                ss[g * kTcTile + key + 1] = key + 1 < nvalid ? s[nt][1] : -INFINITY;
            }
        }
        __syncthreads();

        // ---- online softmax for head g over the 64 keys (every warp computes the same).
        float pv[4][4];  // [k-step][slot pair element]: keys 16*ks + {2t, 2t+1, 2t+8, 2t+9}
        float tmax = -INFINITY;
#pragma unroll
        for (int ks = 0; ks < 4; ks++) {
            const float2 a = *reinterpret_cast<const float2 *>(&ss[g * kTcTile + ks * 16 + 2 * t]);
            const float2 b =
                *reinterpret_cast<const float2 *>(&ss[g * kTcTile + ks * 16 + 2 * t + 8]);
            pv[ks][0] = a.x; pv[ks][1] = a.y; pv[ks][2] = b.x; pv[ks][3] = b.y;
            tmax = fmaxf(tmax, fmaxf(fmaxf(a.x, a.y), fmaxf(b.x, b.y)));
        }
        tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 1));
        tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 2));
        const float m_new = fmaxf(m_run, tmax);
        // m_new is -inf only while every key so far was masked: nothing to scale then.
        const float corr = (m_new == -INFINITY) ? 1.0f : exp2f(m_run - m_new);
        float psum = 0.0f;
#pragma unroll
        for (int ks = 0; ks < 4; ks++)
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const float w = (pv[ks][e] == -INFINITY) ? 0.0f : exp2f(pv[ks][e] - m_new);
                pv[ks][e] = w;
                psum += w;
            }
        psum += __shfl_xor_sync(0xffffffffu, psum, 1);
        psum += __shfl_xor_sync(0xffffffffu, psum, 2);
        l_run = l_run * corr + psum;
        m_run = m_new;
#pragma unroll
        for (int a = 0; a < 2; a++)
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int c = 0; c < 4; c++) acc[a][i][c] *= corr;

        // ---- values: warp w owns blocks 2w, 2w+1 (64 dims) for all 64 keys.
#pragma unroll
        for (int ks = 0; ks < 4; ks++) {
            const int k0 = ks * 16 + 2 * t;  // keys k0, k0+1, k0+8, k0+9
            const unsigned char *r[4] = {vtile[buf] + (k0)*kTcRowBytes,
                                         vtile[buf] + (k0 + 1) * kTcRowBytes,
                                         vtile[buf] + (k0 + 8) * kTcRowBytes,
                                         vtile[buf] + (k0 + 9) * kTcRowBytes};
            const bool ok[4] = {k0 < nvalid, k0 + 1 < nvalid, k0 + 8 < nvalid, k0 + 9 < nvalid};
            // weights scaled by 2^10 and split into f16 high + low
            __half ph[4], pl[4];
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const float w = pv[ks][e] * kPScale;
                ph[e] = __float2half_rn(w);
                pl[e] = __float2half_rn(w - __half2float(ph[e]));
            }
            const __half2 ph01 = __halves2half2(ph[0], ph[1]), ph23 = __halves2half2(ph[2], ph[3]);
            const __half2 pl01 = __halves2half2(pl[0], pl[1]), pl23 = __halves2half2(pl[2], pl[3]);
#pragma unroll
            for (int a = 0; a < 2; a++) {
                const int blk = warp * 2 + a;
                // A = weight * block scale (exact product kept as high + low halves)
                __half dv[4];
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const unsigned short raw =
                        *reinterpret_cast<const unsigned short *>(r[e] + blk * kQ8BlockBytes);
                    dv[e] = ok[e] ? __ushort_as_half(raw) : __ushort_as_half(0);
                }
                const __half2 d01 = __halves2half2(dv[0], dv[1]), d23 = __halves2half2(dv[2], dv[3]);
                const __half2 h01 = __hmul2(ph01, d01), h23 = __hmul2(ph23, d23);
                const __half2 l01 = __hfma2(pl01, d01, __hfma2(ph01, d01, __hneg2(h01)));
                const __half2 l23 = __hfma2(pl23, d23, __hfma2(ph23, d23, __hneg2(h23)));
                unsigned afrag[4];
                afrag[0] = *reinterpret_cast<const unsigned *>(&h01);
                afrag[1] = *reinterpret_cast<const unsigned *>(&l01);
                afrag[2] = *reinterpret_cast<const unsigned *>(&h23);
                afrag[3] = *reinterpret_cast<const unsigned *>(&l23);
                // B: logical word g of the block from each of the four keys
                unsigned w[4];
#pragma unroll
                for (int e = 0; e < 4; e++)
                    w[e] = block_word(reinterpret_cast<const unsigned *>(r[e]), blk, g) ^ 0x80808080u;
                const unsigned ab01 = __byte_perm(w[0], w[1], 0x5140);  // [a0 b0 a1 b1]
                const unsigned ab23 = __byte_perm(w[0], w[1], 0x7362);  // [a2 b2 a3 b3]
                const unsigned cd01 = __byte_perm(w[2], w[3], 0x5140);
                const unsigned cd23 = __byte_perm(w[2], w[3], 0x7362);
                mma_16816(acc[a][0], afrag, codes_to_half2(ab01, 0x4140), codes_to_half2(cd01, 0x4140));
                mma_16816(acc[a][1], afrag, codes_to_half2(ab01, 0x4342), codes_to_half2(cd01, 0x4342));
                mma_16816(acc[a][2], afrag, codes_to_half2(ab23, 0x4140), codes_to_half2(cd23, 0x4140));
                mma_16816(acc[a][3], afrag, codes_to_half2(ab23, 0x4342), codes_to_half2(cd23, 0x4342));
            }
        }
        __syncthreads();  // tile buffers and ss are reused by the next iteration
    }

    // ---- partials: head g's row is c0/c1 (high part) + c2/c3 (low part).
    if (g < group) {
        const int h = kvh * group + g;
        float *pa = p.part_acc + (size_t)slot * p.acc_slot + ((size_t)h * p.splits + split) * 256;
        const float inv = 1.0f / kPScale;
#pragma unroll
        for (int a = 0; a < 2; a++)
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int blk = warp * 2 + a;
                pa[block_word_dim(blk, 2 * t, i)] = (acc[a][i][0] + acc[a][i][2]) * inv;
                pa[block_word_dim(blk, 2 * t + 1, i)] = (acc[a][i][1] + acc[a][i][3]) * inv;
            }
        if (warp == 0 && t == 0) {
            float *pm = p.part_ml + (size_t)slot * p.ml_slot + ((size_t)h * p.splits + split) * 2;
            pm[0] = m_run;
            pm[1] = l_run;
        }
    }
}

}  // namespace

// Entry names and parameter lists of the reduce kernels are the reference's
// (attn_decode_kv.hip:491-496 and its _b form): grid (n_heads[, slots]), block head_dim.
extern "C" __global__ void attn_decode_kv_reduce(const float *__restrict__ part_acc,
                                                 const float *__restrict__ part_ml,
                                                 float *__restrict__ out, int head_dim,
                                                 int splits) {
    const int h = blockIdx.x, d = threadIdx.x;
    if (d >= head_dim) return;
    const float *ml = part_ml + (size_t)h * splits * 2;
    float big = -INFINITY;
    for (int s = 0; s < splits; s++) big = fmaxf(big, ml[2 * s]);
    float num = 0.0f, den = 0.0f;
    for (int s = 0; s < splits; s++) {
        const float m = ml[2 * s];
        const float w = (m == -INFINITY) ? 0.0f : exp2f(m - big);
        num += part_acc[((size_t)h * splits + s) * head_dim + d] * w;
        den += ml[2 * s + 1] * w;
    }
    out[(size_t)h * head_dim + d] = den > 0.0f ? num / den : 0.0f;
}

extern "C" __global__ void attn_decode_kv_reduce_b(const float *__restrict__ part_acc,
                                                   const float *__restrict__ part_ml,
                                                   float *__restrict__ out, int head_dim,
                                                   int splits, int acc_slot, int ml_slot,
                                                   int out_slot) {
    const int slot = blockIdx.y;
    const int h = blockIdx.x, d = threadIdx.x;
    if (d >= head_dim) return;
    const float *pa = part_acc + (size_t)slot * acc_slot;
    const float *ml = part_ml + (size_t)slot * ml_slot + (size_t)h * splits * 2;
    float big = -INFINITY;
    for (int s = 0; s < splits; s++) big = fmaxf(big, ml[2 * s]);
    float num = 0.0f, den = 0.0f;
    for (int s = 0; s < splits; s++) {
        const float m = ml[2 * s];
        const float w = (m == -INFINITY) ? 0.0f : exp2f(m - big);
        num += pa[((size_t)h * splits + s) * head_dim + d] * w;
        den += ml[2 * s + 1] * w;
    }
    out[(size_t)slot * out_slot + (size_t)h * head_dim + d] = den > 0.0f ? num / den : 0.0f;
}

// Host-side launch of the split pass; the reduce is launched by the caller.
int launch_decode_split(cudaStream_t stream, const DecodeParams &p, int slots, bool tensor_core) {
    if (tensor_core) {
        static bool configured[64] = {};
        int dev = 0;
        cudaGetDevice(&dev);
        if (dev >= 0 && dev < 64 && !configured[dev]) {
            cudaError_t e = cudaFuncSetAttribute(attn_decode_kv_tc,
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 kTcSmemBytes);
            if (e != cudaSuccess) return (int)e;
            configured[dev] = true;
        }
        dim3 grid(p.n_kv * p.splits, slots);
        attn_decode_kv_tc<<<grid, kTcThreads, kTcSmemBytes, stream>>>(p);
    } else {
        const int warps = p.n_heads * p.splits;
        dim3 grid((warps + 3) / 4, slots);
        attn_decode_kv_scalar<<<grid, 128, 0, stream>>>(p);
    }
    return launch_status();
}

const void *lookup_decode_kernel(const char *name) {
    if (strcmp(name, "attn_decode_kv_reduce") == 0) return (const void *)attn_decode_kv_reduce;
    if (strcmp(name, "attn_decode_kv_reduce_b") == 0) return (const void *)attn_decode_kv_reduce_b;
    return nullptr;
}

}  // namespace hipml
