// The fold of split-K decode partials, as warp-level pieces shared by the split pass (which
// folds inside the kernel), the stand-alone fold launch and the collect launch of the
// multi-GPU exchange. One warp owns one query head; lane i owns dims [8i, 8i + 8) of a
// head_dim-256 row.
//
// Algebra (crates/hipml-kernels/kernels/attn_decode_kv.hip:491-532): partial s of a head is
// (acc_s, m_s, l_s) with acc_s = sum_k 2^(score_k - m_s) v_k and l_s the sum of the weights;
// the fold is M = max m_s, acc = sum_s 2^(m_s - M) acc_s, l = sum_s 2^(m_s - M) l_s, again a
// partial, so folds nest: groups of eight runs first, then the groups. Every sum runs in slot
// order with explicit fused multiply-adds, so the result does not depend on which CTA
// arrives last nor on which kernel the pieces are inlined into.
#pragma once

#include "params.cuh"

namespace hipml {

struct FoldAcc {
    float a[8];
    float big, den;
};

// Partials of one head at slots first, first + step, ..., `count` of them (<= 32). pa / ml
// point at the head's slot 0. Reads go to L2 (the partials were written by other SMs). The
// loads of a batch of eight partial rows are issued together with the (max, sum) pairs, so a
// group of eight costs one round trip to L2.
__device__ __forceinline__ FoldAcc fold_warp(const float *pa, const float *ml, int first, int step,
                                             int count, int lane) {
    constexpr int kBatch = 8;
    float4 x[kBatch][2];
#pragma unroll
    for (int j = 0; j < kBatch; j++) {
        if (j < count) {
            const float4 *src =
                reinterpret_cast<const float4 *>(pa + (size_t)(first + j * step) * 256 + lane * 8);
            x[j][0] = __ldcg(src);
            x[j][1] = __ldcg(src + 1);
        } else {
            x[j][0] = x[j][1] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        }
    }
    float m = -INFINITY, l = 0.0f;
    if (lane < count) {
        const float2 v = __ldcg(reinterpret_cast<const float2 *>(ml + 2 * (size_t)(first + lane * step)));
        m = v.x;
        l = v.y;
    }
    FoldAcc r;
    r.big = warp_max(m);
    const float w = (m == -INFINITY) ? 0.0f : exp2f(m - r.big);
    const float lw = __fmul_rn(l, w);
    r.den = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; i++) r.a[i] = 0.0f;
    for (int s0 = 0; s0 < count; s0 += kBatch) {
        if (s0 > 0) {
#pragma unroll
            for (int j = 0; j < kBatch; j++) {
                if (s0 + j < count) {
                    const float4 *src = reinterpret_cast<const float4 *>(
                        pa + (size_t)(first + (s0 + j) * step) * 256 + lane * 8);
                    x[j][0] = __ldcg(src);
                    x[j][1] = __ldcg(src + 1);
                } else {
                    x[j][0] = x[j][1] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                }
            }
        }
#pragma unroll
        for (int j = 0; j < kBatch; j++) {
            // (lanes past `count` hold weight 0)
            const float ws = __shfl_sync(0xffffffffu, w, (s0 + j) & 31);
            r.den = __fadd_rn(r.den, __shfl_sync(0xffffffffu, lw, (s0 + j) & 31));
            r.a[0] = fmaf(x[j][0].x, ws, r.a[0]);
            r.a[1] = fmaf(x[j][0].y, ws, r.a[1]);
            r.a[2] = fmaf(x[j][0].z, ws, r.a[2]);
            r.a[3] = fmaf(x[j][0].w, ws, r.a[3]);
            r.a[4] = fmaf(x[j][1].x, ws, r.a[4]);
            r.a[5] = fmaf(x[j][1].y, ws, r.a[5]);
            r.a[6] = fmaf(x[j][1].z, ws, r.a[6]);
            r.a[7] = fmaf(x[j][1].w, ws, r.a[7]);
        }
    }
    return r;
}

// Arrival at a counter with release (this CTA's writes, made visible to the arriving thread by
// the preceding CTA barrier, come first) and acquire (the other arrivals' writes are visible
// afterwards) in one round trip. Returns the count before the arrival.
__device__ __forceinline__ int arrive_acq_rel(int *counter) {
    int prev;
    asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], 1;" : "=r"(prev) : "l"(counter) : "memory");
    return prev;
}

// Writes a folded group back as a partial (slot `at` of the head).
__device__ __forceinline__ void fold_store_partial(float *pa, float *ml, int at, const FoldAcc &f,
                                                   int lane) {
    float4 *dst = reinterpret_cast<float4 *>(pa + (size_t)at * 256 + lane * 8);
    dst[0] = make_float4(f.a[0], f.a[1], f.a[2], f.a[3]);
    dst[1] = make_float4(f.a[4], f.a[5], f.a[6], f.a[7]);
    if (lane == 0) {
        ml[2 * (size_t)at] = f.big;
        ml[2 * (size_t)at + 1] = f.den;
    }
}

// ---- exchange cells ---------------------------------------------------------------------
// A rank's workspace: a 256-byte header { epoch, arrival counter } and a double-buffered
// table cell[2][shards][n_heads][258] of 8-byte cells { value bits, epoch tag }. A cell is
// written and read as ONE 64-bit scalar (single-copy atomic at 8-byte alignment), so a reader
// that sees the tag of this call sees the value that came with it: no fence, no flag.
constexpr int kExchangeHeaderBytes = 256;

__device__ __forceinline__ unsigned long long cell_pack(float value, int tag) {
    return ((unsigned long long)(unsigned)tag << 32) | (unsigned long long)__float_as_uint(value);
}
__device__ __forceinline__ void st_cell(unsigned long long *p, float value, int tag) {
    asm volatile("st.relaxed.sys.global.b64 [%0], %1;" ::"l"(p), "l"(cell_pack(value, tag)) : "memory");
}
// Two adjacent cells (16-byte aligned): a vector of two 64-bit elements, each element atomic.
__device__ __forceinline__ void st_cell2(unsigned long long *p, float v0, float v1, int tag) {
    asm volatile("st.relaxed.sys.global.v2.b64 [%0], {%1, %2};" ::"l"(p), "l"(cell_pack(v0, tag)),
                 "l"(cell_pack(v1, tag))
                 : "memory");
}
__device__ __forceinline__ unsigned long long ld_cell(const unsigned long long *p) {
    unsigned long long v;
    asm volatile("ld.relaxed.sys.global.b64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void ld_cell2(const unsigned long long *p, unsigned long long &a,
                                         unsigned long long &b) {
    asm volatile("ld.relaxed.sys.global.v2.b64 {%0, %1}, [%2];" : "=l"(a), "=l"(b) : "l"(p) : "memory");
}
__device__ __forceinline__ unsigned long long *cell_row(unsigned char *ws, int parity, int shards,
                                                        int n_heads, int shard, int h) {
    unsigned long long *g = reinterpret_cast<unsigned long long *>(ws + kExchangeHeaderBytes);
    return g + (((size_t)parity * shards + shard) * n_heads + h) * 258;
}
__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// The rank that folds head h when the result is divided by head (x.by_head).
__device__ __forceinline__ int exchange_owner(const DecodeParams::Exchange &x, int n_heads, int h) {
    return h / (n_heads / x.shards);
}

// One warp stores head h's folded triple, tagged e, into every rank's table (by_head: into
// the table of the rank that owns the head).
__device__ __forceinline__ void exchange_publish_warp(const DecodeParams::Exchange &x, int n_heads,
                                                      int h, int e, const FoldAcc &f, int lane) {
    const int w_lo = x.by_head ? exchange_owner(x, n_heads, h) : 0;
    const int w_hi = x.by_head ? w_lo + 1 : x.shards;
    for (int w = w_lo; w < w_hi; w++) {
        unsigned long long *row = cell_row(x.ws[w], e & 1, x.shards, n_heads, x.rank, h);
        unsigned long long *dst = row + lane * 8;
        st_cell2(dst, f.a[0], f.a[1], e);
        st_cell2(dst + 2, f.a[2], f.a[3], e);
        st_cell2(dst + 4, f.a[4], f.a[5], e);
        st_cell2(dst + 6, f.a[6], f.a[7], e);
        if (lane == 0) st_cell2(row + 256, f.big, f.den, e);
    }
}

// One warp waits (until `deadline`, a %globaltimer value) for head h's triples of all ranks
// with tag e in this rank's table and folds them in rank order. False when the time ran out.
__device__ __forceinline__ bool exchange_collect_warp(const DecodeParams::Exchange &x, int n_heads,
                                                      int h, int e, unsigned long long deadline,
                                                      int lane, FoldAcc &f) {
    // lane w < shards: the (max, sum) pair of rank w
    float m = -INFINITY, l = 0.0f;
    bool ok = true;
    if (lane < x.shards) {
        const unsigned long long *src = cell_row(x.ws[x.rank], e & 1, x.shards, n_heads, lane, h) + 256;
        for (unsigned i = 0;; i++) {
            unsigned long long a, b;
            ld_cell2(src, a, b);
            if ((int)(a >> 32) == e && (int)(b >> 32) == e) {
                m = __uint_as_float((unsigned)a);
                l = __uint_as_float((unsigned)b);
                break;
            }
            if ((i & 7) == 7) {
                if (global_timer_ns() > deadline) {
                    ok = false;
                    break;
                }
                __nanosleep(64);
            }
        }
    }
    ok = __all_sync(0xffffffffu, ok);
    if (!ok) return false;
    f.big = warp_max(m);
    const float wt = (m == -INFINITY) ? 0.0f : exp2f(m - f.big);
    const float lw = __fmul_rn(l, wt);
    f.den = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; i++) f.a[i] = 0.0f;
    // four ranks per round: their cells are requested together, so a round costs one trip to
    // memory once the peers' stores have landed; the sums still run in rank order
    for (int w0 = 0; w0 < x.shards; w0 += 4) {
        unsigned long long c[4][8];
        unsigned pending = 0;
#pragma unroll
        for (int j = 0; j < 4; j++)
            if (w0 + j < x.shards) pending |= 1u << j;
        for (unsigned i = 0; pending != 0; i++) {
#pragma unroll
            for (int j = 0; j < 4; j++) {
                if (pending & (1u << j)) {
                    const unsigned long long *src =
                        cell_row(x.ws[x.rank], e & 1, x.shards, n_heads, w0 + j, h) + lane * 8;
                    ld_cell2(src, c[j][0], c[j][1]);
                    ld_cell2(src + 2, c[j][2], c[j][3]);
                    ld_cell2(src + 4, c[j][4], c[j][5]);
                    ld_cell2(src + 6, c[j][6], c[j][7]);
                }
            }
#pragma unroll
            for (int j = 0; j < 4; j++) {
                if (pending & (1u << j)) {
                    bool all = true;
#pragma unroll
                    for (int q = 0; q < 8; q++) all = all && (int)(c[j][q] >> 32) == e;
                    if (all) pending &= ~(1u << j);
                }
            }
            if (pending != 0 && (i & 7) == 7) {
                if (global_timer_ns() > deadline) {
                    ok = false;
                    break;
                }
                __nanosleep(64);
            }
        }
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) return false;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            if (w0 + j < x.shards) {
                const float ws = __shfl_sync(0xffffffffu, wt, w0 + j);
                f.den = __fadd_rn(f.den, __shfl_sync(0xffffffffu, lw, w0 + j));
#pragma unroll
                for (int q = 0; q < 8; q++) f.a[q] = fmaf(__uint_as_float((unsigned)c[j][q]), ws, f.a[q]);
            }
        }
    }
    return true;
}

// Output rows of head h from its fold: normalised (optionally gated) or the raw triple.
__device__ __forceinline__ void fold_emit(const DecodeParams &p, int slot, int h, const FoldAcc &f,
                                          int lane, bool normalize) {
    const size_t at = (size_t)slot * p.out_slot + (size_t)h * p.out_head_stride;
    float *o = p.out + at + lane * 8;
    if (normalize) {
        float r[8];
#pragma unroll
        for (int i = 0; i < 8; i++) r[i] = f.den > 0.0f ? __fdiv_rn(f.a[i], f.den) : 0.0f;
        if (p.gate) {
            const float4 *g = reinterpret_cast<const float4 *>(p.gate + at + lane * 8);
            const float4 g0 = g[0], g1 = g[1];
            const float gv[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
#pragma unroll
            for (int i = 0; i < 8; i++) r[i] *= 1.0f / (1.0f + expf(-gv[i]));
        }
        reinterpret_cast<float4 *>(o)[0] = make_float4(r[0], r[1], r[2], r[3]);
        reinterpret_cast<float4 *>(o)[1] = make_float4(r[4], r[5], r[6], r[7]);
    } else {
        // rows of head_dim + 2 floats are only 8-byte aligned
#pragma unroll
        for (int i = 0; i < 4; i++)
            reinterpret_cast<float2 *>(o)[i] = make_float2(f.a[2 * i], f.a[2 * i + 1]);
        if (lane == 0) {
            p.out[at + 256] = f.big;
            p.out[at + 257] = f.den;
        }
    }
}

}  // namespace hipml
