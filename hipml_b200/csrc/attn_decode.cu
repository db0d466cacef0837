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
#include "q8_pack.cuh"

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

// The eight dequantised values (dims 8*sub .. 8*sub+7 of block blk) of one cache row.
__device__ __forceinline__ void load8_quant(const unsigned char *blk_ptr, int sub, bool q4,
                                            float (&x)[8]) {
    const float d = half_bits_to_float(*reinterpret_cast<const unsigned short *>(blk_ptr));
    if (q4) {
        // low (sub < 2) or high nibbles of bytes 8*(sub & 1) .. +7
        const unsigned short *c = reinterpret_cast<const unsigned short *>(blk_ptr + 2 + (sub & 1) * 8);
        const int shift = (sub >> 1) * 4;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const unsigned short w = c[j];
            x[2 * j] = d * ((float)((w >> shift) & 0xf) - 8.0f);
            x[2 * j + 1] = d * ((float)((w >> (8 + shift)) & 0xf) - 8.0f);
        }
    } else {
        const unsigned short *c = reinterpret_cast<const unsigned short *>(blk_ptr + 2 + sub * 8);
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const unsigned short w = c[j];
            x[2 * j] = d * (float)(signed char)(w & 0xff);
            x[2 * j + 1] = d * (float)(signed char)(w >> 8);
        }
    }
}

__global__ void __launch_bounds__(128) attn_decode_kv_scalar(DecodeParams p) {
    griddep_launch();
    griddep_wait();
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
        const size_t row = head_off + (p.q4 ? q4_row_offset(kvh, p.stride, pos, p.head_dim) +
                                                  (size_t)blk * kQ4BlockBytes
                                            : q8_row_offset(kvh, p.stride, pos, p.head_dim) +
                                                  (size_t)blk * kQ8BlockBytes);
        float part = 0.0f;
        if (live) {
            float kx[8];
            load8_quant(p.k + row, sub, p.q4 != 0, kx);
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
            float vx[8];
            load8_quant(p.v + row, sub, p.q4 != 0, vx);
#pragma unroll
            for (int j = 0; j < 8; j++) acc[j] = acc[j] * corr + w * vx[j];
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

// ------------------------------------------------------------ fast reduce
//
// The fold of the split partials used by the launchers. The kernels that keep the
// reference's names below do the same arithmetic with one thread per output element and a
// serial walk over the splits, which costs tens of microseconds at 256 splits; here a CTA
// of 8 warps owns 32 output dims of one head and each warp folds every 8th split.
__global__ void __launch_bounds__(256) attn_decode_fold(FoldParams p) {
    griddep_launch();
    griddep_wait();
    __shared__ float s_max[8];
    __shared__ float s_num[8][32];
    __shared__ float s_den[8];
    const int chunks = p.head_dim >> 5;
    const int h = blockIdx.x / chunks, chunk = blockIdx.x - h * chunks;
    const int slot = blockIdx.y;
    const int dl = threadIdx.x & 31, sg = threadIdx.x >> 5;
    const float *pa = p.acc + (size_t)slot * p.acc_slot + (size_t)h * p.acc_head_stride + chunk * 32 + dl;
    const float *ml = p.ml + (size_t)slot * p.ml_slot + (size_t)h * p.ml_head_stride;
    const int nsplit = p.splits;
    float big = -INFINITY, num = 0.0f, den = 0.0f;
    if (nsplit <= 256) {
        // One (max, sum) pair per thread: the maximum and every run's weight are found with one
        // round of loads, the weights go to shared memory, and the walk over the partial rows
        // below has no exponentials and four loads in flight.
        __shared__ float s_w[256];
        const int s1 = threadIdx.x;
        const float m = s1 < nsplit ? ml[(size_t)s1 * p.ml_split_stride] : -INFINITY;
        const float l = s1 < nsplit ? ml[(size_t)s1 * p.ml_split_stride + 1] : 0.0f;
        big = warp_max(m);
        if (dl == 0) s_max[sg] = big;
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 8; i++) big = fmaxf(big, s_max[i]);
        const float w = (m == -INFINITY) ? 0.0f : exp2f(m - big);
        s_w[s1] = w;
        den = l * w;   // summed over the CTA with the per-warp sums below
        __syncthreads();
        float n0 = 0.0f, n1 = 0.0f, n2 = 0.0f, n3 = 0.0f;
        int s = sg;
        for (; s + 24 < nsplit; s += 32) {
            n0 += pa[(size_t)s * p.acc_split_stride] * s_w[s];
            n1 += pa[(size_t)(s + 8) * p.acc_split_stride] * s_w[s + 8];
            n2 += pa[(size_t)(s + 16) * p.acc_split_stride] * s_w[s + 16];
            n3 += pa[(size_t)(s + 24) * p.acc_split_stride] * s_w[s + 24];
        }
        for (; s < nsplit; s += 8) n0 += pa[(size_t)s * p.acc_split_stride] * s_w[s];
        num = (n0 + n1) + (n2 + n3);
        den = warp_sum(den);
    } else {
        for (int s = sg; s < nsplit; s += 8) big = fmaxf(big, ml[(size_t)s * p.ml_split_stride]);
        if (dl == 0) s_max[sg] = big;
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 8; i++) big = fmaxf(big, s_max[i]);
        for (int s = sg; s < nsplit; s += 8) {
            const float m = ml[(size_t)s * p.ml_split_stride];
            const float w = (m == -INFINITY) ? 0.0f : exp2f(m - big);
            num += pa[(size_t)s * p.acc_split_stride] * w;
            den += ml[(size_t)s * p.ml_split_stride + 1] * w;
        }
    }
    s_num[sg][dl] = num;
    if (dl == 0) s_den[sg] = den;
    __syncthreads();
    if (sg == 0) {
        float n = 0.0f, d = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; i++) {
            n += s_num[i][dl];
            d += s_den[i];
        }
        float *o = p.out + (size_t)slot * p.out_slot + (size_t)h * p.out_head_stride;
        if (p.normalize) {
            float r = d > 0.0f ? n / d : 0.0f;
            if (p.gate) {
                // the output gate of the layer, applied where the row is produced
                const float g = p.gate[(size_t)slot * p.out_slot + (size_t)h * p.out_head_stride +
                                       chunk * 32 + dl];
                r *= 1.0f / (1.0f + expf(-g));
            }
            o[chunk * 32 + dl] = r;
        } else {
            // the folded triple of this shard: acc (unnormalised), then max (log2 units), sum
            o[chunk * 32 + dl] = n;
            if (chunk == 0 && dl == 0) {
                o[p.head_dim] = big;
                o[p.head_dim + 1] = d;
            }
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
    griddep_launch();
    griddep_wait();
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
    griddep_launch();
    griddep_wait();
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

// Host-side launch of the split pass.
int launch_decode_split(cudaStream_t stream, const DecodeParams &p, int slots, bool tensor_core) {
    if (tensor_core) return launch_decode_tc(stream, p, slots);
    const int warps = p.n_heads * p.splits;
    dim3 grid((warps + 3) / 4, slots);
    return launch_pdl(attn_decode_kv_scalar, grid, dim3(128), 0, stream, 1, p);
}

// Host-side launch of the fold.
int launch_decode_fold(cudaStream_t stream, const FoldParams &p, int n_heads, int slots) {
    dim3 grid(n_heads * (p.head_dim >> 5), slots);
    return launch_pdl(attn_decode_fold, grid, dim3(256), 0, stream, 1, p);
}

// The usual case: partials [n_heads][splits][head_dim] / [n_heads][splits][2] -> out[slot][h][d].
int launch_decode_reduce(cudaStream_t stream, const float *part_acc, const float *part_ml,
                         float *out, int n_heads, int head_dim, int splits, int slots,
                         long long acc_slot, long long ml_slot, long long out_slot,
                         const float *gate) {
    FoldParams p;
    p.acc = part_acc;
    p.ml = part_ml;
    p.out = out;
    p.head_dim = head_dim;
    p.splits = splits;
    p.acc_head_stride = (long long)splits * head_dim;
    p.acc_split_stride = head_dim;
    p.ml_head_stride = (long long)splits * 2;
    p.ml_split_stride = 2;
    p.acc_slot = acc_slot;
    p.ml_slot = ml_slot;
    p.out_slot = out_slot;
    p.out_head_stride = head_dim;
    p.normalize = 1;
    p.gate = gate;
    return launch_decode_fold(stream, p, n_heads, slots);
}

int decode_plan_quota_host(const int *lens, int slots, int splits, int share_slots, int n_kv) {
    int total = 0, longest = 0;
    for (int s = 0; s < slots; s++) {
        const int t = (lens[s] + 63) >> 6;
        total += t;
        longest = t > longest ? t : longest;
    }
    auto runs_at = [&](int q) {
        int runs = 0;
        for (int s = 0; s < slots; s++) runs += shared_runs_of((lens[s] + 63) >> 6, q);
        return runs;
    };
    return solve_quota(total, longest, slots, splits, share_slots, n_kv, runs_at);
}

const void *lookup_decode_kernel(const char *name) {
    if (strcmp(name, "attn_decode_kv_reduce") == 0) return (const void *)attn_decode_kv_reduce;
    if (strcmp(name, "attn_decode_kv_reduce_b") == 0) return (const void *)attn_decode_kv_reduce_b;
    return nullptr;
}

}  // namespace hipml
