// Split-K flash-decode over the q8_0 cache, tensor-core body (head_dim 256).
//
// A CTA of 8 warps owns one (KV head, split[, slot]) and streams its rows through a
// three-stage shared-memory ring filled by bulk asynchronous copies (cp.async.bulk, one per
// tensor and tile, completion on an mbarrier): rows are 272 B, 16-byte aligned, and
// consecutive positions of one head are contiguous, so a 64-key tile of K (or V) is one
// linear 17 KB run. One thread issues the copy of tile i+2 as soon as tile i-1 has been
// consumed, so two tiles (70 KB per CTA, two CTAs per SM) are always in flight while the
// third is being computed on. Both contractions run on the tensor cores
// (mma.sync m16n8k16, f16 operands, f32 accumulate) with operands built in registers:
//   * int8 codes are exact in f16. Scores: one byte permute per two codes -- the byte
//     code + 128 under a zero high byte is the f16 subnormal (code + 128) * 2^-24; the offset
//     leaves through the accumulators, which start at -2^-17 * (sum of the query over the
//     block), and the factor 2^-24 when the scores are read. Values: 0x6400 | (code + 128) is
//     1152 + code, minus 1152 (the weights are all positive, so an offset left in the
//     accumulators would cost precision there);
//   * scores: the codes are the A operand (16 keys x 16 dims), the query the B operand as an
//     f16 high and a low part in two chained MMAs, so the block scale multiplies whole
//     accumulator rows; values: the softmax weights are split into f16 high + low parts
//     stacked along M (rows 0..7 high, rows 8..15 low of the same head);
//   * the per-block f16 scales are applied in f32: on the K side to the 32-wide partial dot
//     products, on the V side folded into the weight operand (weight * scale kept as an
//     exact f16 high + low pair).
// Results agree with the f32 definition to ~1e-6. The CUDA cores only unpack bytes: at 12
// f32 FMA per cache byte a scalar kernel cannot keep up with HBM3e.
//
// Per tile: (1) scores -- warp (kg, dh) computes the partial scores of keys [16kg, 16kg+16)
// over blocks [4dh, 4dh+4); (2) softmax -- warp g owns query head g of the group: running
// max / sum, weights written once to shared memory as f16 high/low; (3) values -- warp w
// owns block w (32 dims) for all 64 keys. CPU definition: crates/hipml-core/src/ops.rs:
// 449-518; kernel replaced: crates/hipml-kernels/kernels/attn_decode_kv_w.hip:92-285 and
// attn_decode_kv.hip:251-374,427-484.
#include <atomic>
#include <map>
#include <mutex>
#include <tuple>

#include "params.cuh"
#include "q8_pack.cuh"
#include "sm100_ptx.cuh"
#include "decode_fold.cuh"

namespace hipml {

namespace {

constexpr int kTile = 64;                        // keys per shared-memory tile
constexpr int kRowBytes = 8 * kQ8BlockBytes;     // 272
constexpr int kTileBytes = kTile * kRowBytes;    // 17408
constexpr int kThreads = 256;
constexpr int kSsStride = 68;                    // padded row of the score tile (floats)
constexpr int kPStride = 72;                     // padded row of the weight tile (halves)
constexpr float kPScale = 1024.0f;               // keeps weight*scale in f16's normal range

constexpr int kStages = 3;                       // ring depth (tiles of K and V)
constexpr unsigned kSpinLimit = 1u << 24;        // polls of a full barrier before giving up

// Dynamic shared memory: stage[3] = (K tile | V tile) | scores [2][8][72] f32 | weights hi,
// lo [8][72] f16 | corr[8] f32 | full barriers [3].
constexpr int kOffSs = 2 * kStages * kTileBytes;
constexpr int kOffPh = kOffSs + 2 * 8 * kSsStride * 4;
constexpr int kOffPl = kOffPh + 8 * kPStride * 2;
constexpr int kOffCorr = kOffPl + 8 * kPStride * 2;
constexpr int kOffBar = kOffCorr + 8 * 4;
constexpr int kSmemBytes = kOffBar + kStages * 8;
static_assert(2 * (kSmemBytes + 1024) <= 227 * 1024, "two CTAs per SM");

using namespace ptx;

__device__ __forceinline__ void mma_16816(float (&c)[4], const unsigned (&a)[4], unsigned b0,
                                          unsigned b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// K side: the eight "logical words" (four codes each) of block blk, all 4-byte aligned loads.
// Odd blocks start 2 bytes past a word boundary, so word j holds codes 4j..4j+3. Even blocks
// start on a word boundary (the scale shares a word with codes 0,1): words 0..6 hold codes
// 4j+2..4j+5 and word 7 is stitched from codes 0,1 and 30,31. The order of elements inside
// the contraction is free as long as the query operand uses the same one.
template <int BLK, int KK>
__device__ __forceinline__ unsigned k_word(const unsigned *row, int t) {
    constexpr int m = BLK >> 1;
    if constexpr (BLK & 1) {
        return row[17 * m + 9 + KK * 4 + t];
    } else if constexpr (KK == 0) {
        return row[17 * m + 1 + t];
    } else {
        // j = 4 + t; j == 7 is the stitched word. Branch-free: two loads and a permute.
        const bool last = t == 3;
        const unsigned a = row[last ? 17 * m : 17 * m + 5 + t];
        const unsigned b = row[last ? 17 * m + 8 : 17 * m + 5 + t];
        return __byte_perm(a, b, last ? 0x5432 : 0x3210);
    }
}

// head_dim index of byte i of logical word j of block blk, in k_word's order.
__device__ __forceinline__ int k_word_dim(int blk, int j, int i) {
    if (blk & 1) return blk * 32 + 4 * j + i;
    if (j < 7) return blk * 32 + 4 * j + 2 + i;
    return blk * 32 + (i < 2 ? i : 28 + i);
}

// V side: codes 4j..4j+3 of a block in natural order; `blk_row` points at the block's first
// aligned word (odd blocks: its first code word; even blocks: the word that starts with the
// scale, so the codes straddle word boundaries: two loads and a permute).
template <bool kOdd>
__device__ __forceinline__ unsigned v_word(const unsigned *blk_row, int j) {
    if constexpr (kOdd) return blk_row[j];
    return __byte_perm(blk_row[j], blk_row[j + 1], 0x5432);
}

// Two bytes of `biased` (code ^ 0x80 = code + 128) as a half2 of f16 subnormals: 0x00xx is
// xx * 2^-24 exactly, so one permute converts two codes. The offset of 128 is taken out
// again through the accumulators (see score_block and the values phase), the factor 2^-24
// when the scores / partials are written.
__device__ __forceinline__ unsigned codes_to_half2(unsigned biased, unsigned selector) {
    return __byte_perm(biased, 0u, selector);
}
// Value side: bytes of `biased` as an exact half2 through 0x64xx = 1024 + xx, minus 1152. The
// weights are all positive there, so an offset carried in the accumulators would cost
// several bits (measured: 4e-5 relative on a flat 256-key run); this form is exact.
__device__ __forceinline__ unsigned codes_to_half2_exact(unsigned biased, unsigned selector) {
    const unsigned h = __byte_perm(biased, 0x64646464u, selector);
    const __half2 r =
        __hsub2(*reinterpret_cast<const __half2 *>(&h), __half2half2(__ushort_as_half(0x6480)));
    return *reinterpret_cast<const unsigned *>(&r);
}
constexpr float kCodeUnit = 16777216.0f;          // 2^24
constexpr float kCodeBias = 128.0f / 16777216.0f; // the offset in the operand's units: 2^-17

__device__ __forceinline__ unsigned pack_half2(__half lo, __half hi) {
    const __half2 r = __halves2half2(lo, hi);
    return *reinterpret_cast<const unsigned *>(&r);
}

// Rows [lo, hi) of run `split` of a slot. The partials are scratch (only their fold is
// defined), so the rows are dealt out for this device (plan_runs): one round of long runs,
// balanced to within one 64-key tile, for a single stream; runs in proportion to the live
// lengths for several slots. Without a plan (more than 64 slots) the reference's runs of
// ceil(capacity / splits) rows apply, rounded up to whole tiles so that no run ends in a
// mostly empty one; runs past the live length get no rows and write neutral partials.
// `runs`: the partial slots of a head that the fold reads (never less than one: a slot without
// rows keeps run 0, which writes a neutral partial, so that its output rows are written).
__device__ __forceinline__ int live_runs(const DecodeParams &p, int slot, int quota) {
    const RunPlan plan = plan_runs(p.len, p.len_stride, p.len_offset, slot, p.splits,
                                   p.by_stride ? 0 : p.run_cap, p.share_slots, quota);
    return plan.runs < 0 ? p.splits : max(plan.runs, 1);
}
__device__ __forceinline__ void split_range(const DecodeParams &p, int slot, int split, int quota,
                                            int &lo, int &hi) {
    const int len = p.len[slot * p.len_stride + p.len_offset];
    const RunPlan plan = plan_runs(p.len, p.len_stride, p.len_offset, slot, p.splits,
                                   p.by_stride ? 0 : p.run_cap, p.share_slots, quota);
    if (plan.runs >= 0) {
        if (split >= plan.runs) {
            lo = hi = len;
            return;
        }
        lo = (int)((long long)split * plan.tiles / plan.runs) * kTile;
        hi = min((int)((long long)(split + 1) * plan.tiles / plan.runs) * kTile, len);
        return;
    }
    const int span = p.by_stride ? p.stride : len;
    const int per = ((span + p.splits - 1) / p.splits + kTile - 1) / kTile * kTile;
    lo = min(split * per, len);
    hi = min(lo + per, len);
}

// Scores of one block for this warp's 16 keys, added into s. The codes are the A operand
// (rows = keys g and g + 8 of the 16, contraction slots in k_word's order), the query the B
// operand (columns = heads), so the block scale is one factor per accumulator row:
// s[0], s[1] = key g, heads 2t and 2t + 1; s[2], s[3] = key g + 8. The accumulators start at
// -2^-17 * (sum of the head's query over the block), which removes the codes' offset of 128.
template <int BLK>
__device__ __forceinline__ void score_block(const unsigned char *ktile, int key_base, int g, int t,
                                            const unsigned (&qb0)[4], const unsigned (&qb1)[4],
                                            const float (&bias)[2], float (&s)[4]) {
    const unsigned *row0 = reinterpret_cast<const unsigned *>(ktile + (key_base + g) * kRowBytes);
    const unsigned *row1 = row0 + 8 * (kRowBytes / 4);
    float c[4] = {bias[0], bias[1], bias[0], bias[1]};
    {
        const unsigned w0 = k_word<BLK, 0>(row0, t) ^ 0x80808080u;
        const unsigned w1 = k_word<BLK, 0>(row1, t) ^ 0x80808080u;
        const unsigned a[4] = {codes_to_half2(w0, 0x4140), codes_to_half2(w1, 0x4140),
                               codes_to_half2(w0, 0x4342), codes_to_half2(w1, 0x4342)};
        mma_16816(c, a, qb0[0], qb0[1]);
        mma_16816(c, a, qb0[2], qb0[3]);
    }
    {
        const unsigned w0 = k_word<BLK, 1>(row0, t) ^ 0x80808080u;
        const unsigned w1 = k_word<BLK, 1>(row1, t) ^ 0x80808080u;
        const unsigned a[4] = {codes_to_half2(w0, 0x4140), codes_to_half2(w1, 0x4140),
                               codes_to_half2(w0, 0x4342), codes_to_half2(w1, 0x4342)};
        mma_16816(c, a, qb1[0], qb1[1]);
        mma_16816(c, a, qb1[2], qb1[3]);
    }
    const unsigned char *sc = ktile + (key_base + g) * kRowBytes + BLK * kQ8BlockBytes;
    const float d0 = half_bits_to_float(*reinterpret_cast<const unsigned short *>(sc));
    const float d1 = half_bits_to_float(*reinterpret_cast<const unsigned short *>(sc + 8 * kRowBytes));
    s[0] += d0 * c[0];
    s[1] += d0 * c[1];
    s[2] += d1 * c[2];
    s[3] += d1 * c[3];
}

// Values of one tile for block `blk` (32 dims): acc = acc * corr + weights * scale * codes over
// the 64 keys. A = weight * block scale as an exact f16 high + low pair (rows 0..7 high part of
// head g, rows 8..15 low part), B = the block's codes, four n-tiles: output column n of MMA i
// is dim 32*blk + 4n + i. All shared-memory offsets inside the unrolled loop are immediates
// off three per-thread base pointers.
template <bool kOdd>
__device__ __forceinline__ void values_block(const unsigned char *vtile, int blk, int g, int t,
                                             const __half *ph, const __half *pl, float corr,
                                             float (&acc)[4][4]) {
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int c = 0; c < 4; c++) acc[i][c] *= corr;
    // keys k0 = 16*ks + 2t, k0 + 1, k0 + 8, k0 + 9 of every 16-key step
    const unsigned char *scale0 = vtile + 2 * t * kRowBytes + blk * kQ8BlockBytes;
    const unsigned *code0 =
        reinterpret_cast<const unsigned *>(scale0 + (kOdd ? 2 : 0)) + g;
    const __half *ph0 = ph + g * kPStride + 2 * t, *pl0 = pl + g * kPStride + 2 * t;
    constexpr int kRowWords = kRowBytes / 4;
#pragma unroll
    for (int ks = 0; ks < 4; ks++) {
        constexpr int kOff[4] = {0, 1, 8, 9};
        __half dv[4];
        unsigned w[4];
#pragma unroll
        for (int e = 0; e < 4; e++) {
            dv[e] = __ushort_as_half(*reinterpret_cast<const unsigned short *>(
                scale0 + (ks * 16 + kOff[e]) * kRowBytes));
            w[e] = v_word<kOdd>(code0 + (ks * 16 + kOff[e]) * kRowWords, 0) ^ 0x80808080u;
        }
        const __half2 d01 = __halves2half2(dv[0], dv[1]), d23 = __halves2half2(dv[2], dv[3]);
        const __half2 ph01 = *reinterpret_cast<const __half2 *>(ph0 + ks * 16);
        const __half2 ph23 = *reinterpret_cast<const __half2 *>(ph0 + ks * 16 + 8);
        const __half2 pl01 = *reinterpret_cast<const __half2 *>(pl0 + ks * 16);
        const __half2 pl23 = *reinterpret_cast<const __half2 *>(pl0 + ks * 16 + 8);
        const __half2 h01 = __hmul2(ph01, d01), h23 = __hmul2(ph23, d23);
        const __half2 l01 = __hfma2(pl01, d01, __hfma2(ph01, d01, __hneg2(h01)));
        const __half2 l23 = __hfma2(pl23, d23, __hfma2(ph23, d23, __hneg2(h23)));
        unsigned afrag[4];
        afrag[0] = *reinterpret_cast<const unsigned *>(&h01);
        afrag[1] = *reinterpret_cast<const unsigned *>(&l01);
        afrag[2] = *reinterpret_cast<const unsigned *>(&h23);
        afrag[3] = *reinterpret_cast<const unsigned *>(&l23);
        const unsigned ab01 = __byte_perm(w[0], w[1], 0x5140);  // [a0 b0 a1 b1]
        const unsigned ab23 = __byte_perm(w[0], w[1], 0x7362);  // [a2 b2 a3 b3]
        const unsigned cd01 = __byte_perm(w[2], w[3], 0x5140);
        const unsigned cd23 = __byte_perm(w[2], w[3], 0x7362);
        mma_16816(acc[0], afrag, codes_to_half2_exact(ab01, 0x4140), codes_to_half2_exact(cd01, 0x4140));
        mma_16816(acc[1], afrag, codes_to_half2_exact(ab01, 0x4342), codes_to_half2_exact(cd01, 0x4342));
        mma_16816(acc[2], afrag, codes_to_half2_exact(ab23, 0x4140), codes_to_half2_exact(cd23, 0x4140));
        mma_16816(acc[3], afrag, codes_to_half2_exact(ab23, 0x4342), codes_to_half2_exact(cd23, 0x4342));
    }
}

// ---- q4_0 rows read in place (144-byte rows of 18-byte blocks: f16 scale, then 16 bytes
// whose low nibbles are values 0..15 and high nibbles values 16..31, each value + 8).
constexpr int kQ4RowBytes = 8 * kQ4BlockBytes;   // 144 = 36 words; a block pair is 9 words

// K side: the four "logical words" of block BLK (four code bytes each), aligned loads only.
// Odd blocks start on a word boundary after their scale's half word; even blocks hold bytes
// 2..13 in three aligned words and bytes 0, 1, 14, 15 in the two words they share with the
// scales, stitched into the fourth. The contraction order is free (the query follows it).
template <int BLK>
__device__ __forceinline__ unsigned k_word_q4(const unsigned *row, int t) {
    constexpr int m = BLK >> 1;
    if constexpr (BLK & 1) {
        return row[9 * m + 5 + t];
    } else {
        const bool last = t == 3;
        const unsigned a = row[last ? 9 * m : 9 * m + 1 + t];
        const unsigned b = row[last ? 9 * m + 4 : 9 * m + 1 + t];
        return __byte_perm(a, b, last ? 0x5432 : 0x3210);
    }
}
// head_dim index of byte i of logical word j (low nibble; the high nibble is 16 further).
__device__ __forceinline__ int k_word_dim_q4(int blk, int j, int i) {
    if (blk & 1) return blk * 32 + 4 * j + i;
    if (j < 3) return blk * 32 + 4 * j + 2 + i;
    return blk * 32 + (i < 2 ? i : 12 + i);
}

// Scores of one q4_0 block for this warp's 16 keys: as score_block, with step 0 of the
// contraction over the low nibbles (values 0..15 of the block) and step 1 over the high ones.
// A nibble is value + 8, an f16 subnormal as it stands: no XOR, offset 8.
template <int BLK>
__device__ __forceinline__ void score_block_q4(const unsigned char *ktile, int key_base, int g, int t,
                                               const unsigned (&qb0)[4], const unsigned (&qb1)[4],
                                               const float (&bias)[2], float (&s)[4]) {
    const unsigned *row0 = reinterpret_cast<const unsigned *>(ktile + (key_base + g) * kQ4RowBytes);
    const unsigned *row1 = row0 + 8 * (kQ4RowBytes / 4);
    float c[4] = {bias[0], bias[1], bias[0], bias[1]};
    const unsigned w0 = k_word_q4<BLK>(row0, t), w1 = k_word_q4<BLK>(row1, t);
    {
        const unsigned x0 = w0 & 0x0f0f0f0fu, x1 = w1 & 0x0f0f0f0fu;
        const unsigned a[4] = {codes_to_half2(x0, 0x4140), codes_to_half2(x1, 0x4140),
                               codes_to_half2(x0, 0x4342), codes_to_half2(x1, 0x4342)};
        mma_16816(c, a, qb0[0], qb0[1]);
        mma_16816(c, a, qb0[2], qb0[3]);
    }
    {
        const unsigned x0 = (w0 >> 4) & 0x0f0f0f0fu, x1 = (w1 >> 4) & 0x0f0f0f0fu;
        const unsigned a[4] = {codes_to_half2(x0, 0x4140), codes_to_half2(x1, 0x4140),
                               codes_to_half2(x0, 0x4342), codes_to_half2(x1, 0x4342)};
        mma_16816(c, a, qb1[0], qb1[1]);
        mma_16816(c, a, qb1[2], qb1[3]);
    }
    const unsigned char *sc = ktile + (key_base + g) * kQ4RowBytes + BLK * kQ4BlockBytes;
    const float d0 = half_bits_to_float(*reinterpret_cast<const unsigned short *>(sc));
    const float d1 = half_bits_to_float(*reinterpret_cast<const unsigned short *>(sc + 8 * kQ4RowBytes));
    s[0] += d0 * c[0];
    s[1] += d0 * c[1];
    s[2] += d1 * c[2];
    s[3] += d1 * c[3];
}

// Values of one tile for q4_0 block `blk`: as values_block. Lane group g takes code word g & 3
// (natural order: values 4(g&3) .. +3 in the low nibbles, 16 further in the high ones) and the
// nibble half g >> 2, so output column n of MMA i is dim 32*blk + 4n + i as for q8_0.
// 0x6400 | nibble is 1024 + value + 8, minus 1032: exact.
template <bool kOdd>
__device__ __forceinline__ void values_block_q4(const unsigned char *vtile, int blk, int g, int t,
                                                const __half *ph, const __half *pl, float corr,
                                                float (&acc)[4][4]) {
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int c = 0; c < 4; c++) acc[i][c] *= corr;
    const unsigned char *scale0 = vtile + 2 * t * kQ4RowBytes + blk * kQ4BlockBytes;
    const unsigned *code0 = reinterpret_cast<const unsigned *>(scale0 + (kOdd ? 2 : 0)) + (g & 3);
    const int shift = (g >> 2) * 4;
    const __half *ph0 = ph + g * kPStride + 2 * t, *pl0 = pl + g * kPStride + 2 * t;
    constexpr int kRowWords = kQ4RowBytes / 4;
    const __half2 off = __half2half2(__ushort_as_half(0x6408));   // 1032
#pragma unroll
    for (int ks = 0; ks < 4; ks++) {
        constexpr int kOff[4] = {0, 1, 8, 9};
        __half dv[4];
        unsigned w[4];
#pragma unroll
        for (int e = 0; e < 4; e++) {
            dv[e] = __ushort_as_half(*reinterpret_cast<const unsigned short *>(
                scale0 + (ks * 16 + kOff[e]) * kQ4RowBytes));
            w[e] = (v_word<kOdd>(code0 + (ks * 16 + kOff[e]) * kRowWords, 0) >> shift) & 0x0f0f0f0fu;
        }
        const __half2 d01 = __halves2half2(dv[0], dv[1]), d23 = __halves2half2(dv[2], dv[3]);
        const __half2 ph01 = *reinterpret_cast<const __half2 *>(ph0 + ks * 16);
        const __half2 ph23 = *reinterpret_cast<const __half2 *>(ph0 + ks * 16 + 8);
        const __half2 pl01 = *reinterpret_cast<const __half2 *>(pl0 + ks * 16);
        const __half2 pl23 = *reinterpret_cast<const __half2 *>(pl0 + ks * 16 + 8);
        const __half2 h01 = __hmul2(ph01, d01), h23 = __hmul2(ph23, d23);
        const __half2 l01 = __hfma2(pl01, d01, __hfma2(ph01, d01, __hneg2(h01)));
        const __half2 l23 = __hfma2(pl23, d23, __hfma2(ph23, d23, __hneg2(h23)));
        unsigned afrag[4];
        afrag[0] = *reinterpret_cast<const unsigned *>(&h01);
        afrag[1] = *reinterpret_cast<const unsigned *>(&l01);
        afrag[2] = *reinterpret_cast<const unsigned *>(&h23);
        afrag[3] = *reinterpret_cast<const unsigned *>(&l23);
        const unsigned ab01 = __byte_perm(w[0], w[1], 0x5140);  // [a0 b0 a1 b1]
        const unsigned ab23 = __byte_perm(w[0], w[1], 0x7362);  // [a2 b2 a3 b3]
        const unsigned cd01 = __byte_perm(w[2], w[3], 0x5140);
        const unsigned cd23 = __byte_perm(w[2], w[3], 0x7362);
        auto conv = [&](unsigned x, unsigned sel) {
            const unsigned h = __byte_perm(x, 0x64646464u, sel);
            const __half2 r = __hsub2(*reinterpret_cast<const __half2 *>(&h), off);
            return *reinterpret_cast<const unsigned *>(&r);
        };
        mma_16816(acc[0], afrag, conv(ab01, 0x4140), conv(cd01, 0x4140));
        mma_16816(acc[1], afrag, conv(ab01, 0x4342), conv(cd01, 0x4342));
        mma_16816(acc[2], afrag, conv(ab23, 0x4140), conv(cd23, 0x4140));
        mma_16816(acc[3], afrag, conv(ab23, 0x4342), conv(cd23, 0x4342));
    }
}

// Arrival counters of the fold inside the split pass: kArriveRegions regions of
// kArriveRegionInts counters, zero at load and zero again after every launch that used them.
constexpr int kArriveRegions = 128;
__device__ int g_arrive[kArriveRegions * kArriveRegionInts];

// What the CTA that holds the final fold of a (slot, KV head) does with it: write the output
// rows, or (sequence-split decode across GPUs) publish the triples to every rank's table
// and / or collect all ranks' triples and fold those. All threads of the CTA call it; warp w
// holds head w of the group in f.
__device__ __forceinline__ void fold_finish(const DecodeParams &p, int *status, int slot, int kvh,
                                            int group, FoldAcc &f) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int h = kvh * group + warp;
    if (p.xch.phases == 0) {
        if (warp < group) fold_emit(p, slot, h, f, lane, p.normalize != 0);
        return;
    }
    __shared__ int s_epoch;
    int *hdr = reinterpret_cast<int *>(p.xch.ws[p.xch.rank]);
    // Every folding CTA of the call reads the epoch before it adds itself to the counter, and
    // the epoch advances only after the last of them has: all of them see the same value.
    if (threadIdx.x == 0) s_epoch = *reinterpret_cast<volatile int *>(hdr) + ((p.xch.phases & 1) ? 1 : 0);
    __syncthreads();
    const int e = s_epoch;
    if (p.xch.phases & 1) {
        if (warp < group) exchange_publish_warp(p.xch, p.n_heads, h, e, f, lane);
        __syncthreads();
        if (threadIdx.x == 0) {
            if (atomicAdd(hdr + 1, 1) == p.n_kv - 1) {
                hdr[1] = 0;
                *reinterpret_cast<volatile int *>(hdr) = e;
            }
        }
    }
    if (p.xch.phases & 2) {
        if (warp < group && (!p.xch.by_head || exchange_owner(p.xch, p.n_heads, h) == p.xch.rank)) {
            const unsigned long long deadline = global_timer_ns() + 1000ull * p.xch.wait_us;
            if (exchange_collect_warp(p.xch, p.n_heads, h, e, deadline, lane, f))
                fold_emit(p, slot, h, f, lane, true);
            else if (lane == 0 && status)
                atomicCAS(status, 0, 31);
        }
    }
}

// The end of a split-pass CTA whose partial is live: arrive at the group's counter; the last
// of a group folds it into the group's first slot and arrives at the head group's counter;
// the last of those folds the groups and finishes. Nobody waits: whoever is not last is done.
__device__ __forceinline__ void fold_tail(const DecodeParams &p, int *status, int slot, int kvh,
                                          int split, int runs, int group, int tid) {
    __shared__ int s_role;
    const int warp = tid >> 5, lane = tid & 31;
    const int gsize = fold_group_of(runs);
    const int ngroups = (runs + gsize - 1) / gsize;
    const int grp = split / gsize;
    const int expect = min(gsize, runs - grp * gsize);
    int *ctr = g_arrive + (size_t)p.arrive_region * kArriveRegionInts +
               (size_t)(slot * p.n_kv + kvh) * p.arrive_stride;
    // (every thread's partial stores precede the barrier; the arrival releases them)
    __syncthreads();
    if (tid == 0) {
        int role = 1;
        if (expect > 1) {
            role = arrive_acq_rel(ctr + 1 + grp) == expect - 1;
            if (role) ctr[1 + grp] = 0;
        }
        s_role = role;
    }
    __syncthreads();
    if (!s_role) return;
    const int h = kvh * group + warp;
    float *pa = p.part_acc + (size_t)slot * p.acc_slot + (size_t)h * p.splits * 256;
    float *ml = p.part_ml + (size_t)slot * p.ml_slot + (size_t)h * p.splits * 2;
    FoldAcc f;
    if (warp < group) f = fold_warp(pa, ml, grp * gsize, 1, expect, lane);
    if (ngroups > 1) {
        if (warp < group) fold_store_partial(pa, ml, grp * gsize, f, lane);
        __syncthreads();
        if (tid == 0) {
            const int role = arrive_acq_rel(ctr) == ngroups - 1;
            if (role) ctr[0] = 0;
            s_role = role;
        }
        __syncthreads();
        if (!s_role) return;
        if (warp < group) f = fold_warp(pa, ml, 0, gsize, ngroups, lane);
    }
    fold_finish(p, status, slot, kvh, group, f);
}

// kQ4: the cache is q4_0; the phases read the 144-byte rows as they were copied.
template <bool kQ4>
__global__ void __launch_bounds__(kThreads, 2) attn_decode_kv_tc(DecodeParams p, int *status) {
    extern __shared__ __align__(16) unsigned char smem[];
    griddep_launch();
    // Everything this kernel reads -- the live lengths, the query, the cache rows with this
    // step's append -- may come from the grids before it, and a dependent launch can start
    // while the grid before its predecessor is still running: nothing is read before this.
    griddep_wait();
    auto ktile_at = [&](int stage) { return smem + 2 * stage * kTileBytes; };
    auto vtile_at = [&](int stage) { return smem + (2 * stage + 1) * kTileBytes; };
    float *ss = reinterpret_cast<float *>(smem + kOffSs);            // [2][8][kSsStride]
    __half *ph = reinterpret_cast<__half *>(smem + kOffPh);          // [8][kPStride]
    __half *pl = reinterpret_cast<__half *>(smem + kOffPl);
    float *corr_s = reinterpret_cast<float *>(smem + kOffCorr);      // [8]

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int group = p.n_heads / p.n_kv;
    const int kg = warp & 3, dh = warp >> 2;

    // Which (slot, KV head, run) this CTA owns. Plain form: grid (n_kv * splits, slots).
    // Shared form (several slots, share_slots > 0): a one-dimensional grid of exactly the
    // device's CTA slots; CTA b takes the b-th live run in (slot, head, run) order, found by a
    // scan over the slots' run counts, and CTAs past the last live run have nothing to do (no
    // dead run is ever launched, so no live run waits behind them).
    __shared__ int s_plan[4];   // slot (-1: none), kvh, split, quota
    // (single stream with balanced runs: only the first min(splits, run_cap) runs of a head
    // can hold rows, and only those are launched)
    const int grid_splits = (p.by_stride || p.run_cap <= 0) ? p.splits : min(p.splits, p.run_cap);
    int slot = blockIdx.y, kvh = blockIdx.x / grid_splits, split = blockIdx.x - kvh * grid_splits;
    if (p.share_slots > 0) {
        if (warp == 0) {
            const int quota = shared_quota_warp(p.len, p.len_stride, p.len_offset, p.n_slots, p.splits,
                                                p.share_slots, p.n_kv);
            const int b = blockIdx.x;
            int base = 0;
            if (lane == 0) {
                s_plan[0] = -1;
                s_plan[3] = quota;
            }
            __syncwarp();
            for (int s0 = 0; s0 < p.n_slots; s0 += 32) {
                const int s = s0 + lane;
                const int per = s < p.n_slots
                    ? shared_runs_of((p.len[s * p.len_stride + p.len_offset] + 63) >> 6, quota) : 0;
                const int runs = per * p.n_kv;
                int incl = runs;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const int up = __shfl_up_sync(0xffffffffu, incl, o);
                    if (lane >= o) incl += up;
                }
                const int first = base + incl - runs;
                if (runs > 0 && b >= first && b < first + runs) {
                    const int r = b - first;
                    s_plan[0] = s;
                    s_plan[1] = r / per;
                    s_plan[2] = r - (r / per) * per;
                }
                base += __shfl_sync(0xffffffffu, incl, 31);
            }
        }
        __syncthreads();
        slot = s_plan[0];
        kvh = s_plan[1];
        split = s_plan[2];
        if (slot < 0) return;
    }
    // The query values this lane feeds to the tensor cores, loaded straight into registers
    // before anything that depends on the live length, so that the two round trips overlap.
    float qv[8][4];
    {
        const float *qh = p.q + (size_t)slot * p.q_slot + (size_t)(kvh * group + g) * 256;
#pragma unroll
        for (int ks = 0; ks < 8; ks++) {
            const int blk = dh * 4 + (ks >> 1), j = (ks & 1) * 4 + t;
#pragma unroll
            for (int i = 0; i < 4; i += 2) {
                const int d = kQ4 ? k_word_dim_q4(blk, t, i) + 16 * (ks & 1) : k_word_dim(blk, j, i);
                float2 x = make_float2(0.0f, 0.0f);
                if (g < group) x = *reinterpret_cast<const float2 *>(qh + d);
                qv[ks][i] = x.x;
                qv[ks][i + 1] = x.y;
            }
        }
    }
    int lo, hi;
    split_range(p, slot, split, p.share_slots > 0 ? s_plan[3] : 0, lo, hi);
    const int ntiles = (hi - lo + kTile - 1) / kTile;
    if (ntiles == 0) {
        // A split without rows: neutral partials (zero sum, -inf maximum), nothing else.
        for (int i = tid; i < group * 256; i += kThreads) {
            const int h = kvh * group + (i >> 8);
            p.part_acc[(size_t)slot * p.acc_slot + ((size_t)h * p.splits + split) * 256 + (i & 255)] = 0.0f;
        }
        if (tid < group) {
            float *pm = p.part_ml + (size_t)slot * p.ml_slot +
                        ((size_t)(kvh * group + tid) * p.splits + split) * 2;
            pm[0] = -INFINITY;
            pm[1] = 0.0f;
        }
    }

    if (ntiles > 0) {
    constexpr int kSrcRow = kQ4 ? kQ4RowBytes : kRowBytes;   // bytes of a cache row
    const size_t head_byte = (size_t)slot * p.kv_slot_bytes + (size_t)kvh * p.stride * kSrcRow;
    const unsigned char *kbase = p.k + head_byte;
    const unsigned char *vbase = p.v + head_byte;
    int append_pos = -1;
    if (p.k_row != nullptr) {
        append_pos = p.len[slot * p.len_stride + p.len_offset - 1];
        // the fused form appends the last live row; anything else is the caller's error
        if (split == 0 && kvh == 0 && tid == 0 &&
            append_pos != p.len[slot * p.len_stride + p.len_offset] - 1 && status)
            atomicCAS(status, 0, 22);
    }

    // Ring: stage tile % 3; thread 0 arms the stage's barrier with the byte count and issues
    // the two copies. A stage is re-filled only after the __syncthreads that ends the tile
    // which last read it.
    const unsigned bar_full = smem_u32(smem + kOffBar);
    auto fetch = [&](int tile) {
        const int stage = tile % kStages;
        const int r0 = lo + tile * kTile;
        const unsigned bytes = (unsigned)(min(kTile, hi - r0) * kSrcRow);
        const size_t off = (size_t)r0 * kSrcRow;
        constexpr int kDst = 0;
        // earlier generic-proxy writes to the stage (the zero fill of a short tile) come first
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        mbar_arrive_expect_tx(bar_full + 8 * stage, 2 * bytes);
        bulk_load(smem_u32(ktile_at(stage)) + kDst, kbase + off, bytes, bar_full + 8 * stage);
        bulk_load(smem_u32(vtile_at(stage)) + kDst, vbase + off, bytes, bar_full + 8 * stage);
    };
    if (tid == 0) {
#pragma unroll
        for (int s = 0; s < kStages; s++) mbar_init(bar_full + 8 * s, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fetch(0);
        if (ntiles > 1) fetch(1);
    }

    // B fragments of the query for this warp's four blocks and both 16-slot steps of each:
    // column g = head g, as an f16 high and low part ({hi b0, hi b1, lo b0, lo b1}); the
    // contraction slots follow k_word's order (slots 2t, 2t+1 = bytes 0, 1 of word t, slots
    // 2t+8, 2t+9 = bytes 2, 3). The 32 values a lane needs arrived in registers (qv, loaded
    // straight from memory in that order while the first tiles were being fetched); rows past
    // the group are zero. Scores are kept in log2 units.
    unsigned qb[8][4];
    float qbias[4][2];
#pragma unroll
    for (int b = 0; b < 4; b++) {
        float sum = 0.0f;   // of the block's query values as the tensor cores see them
#pragma unroll
        for (int half = 0; half < 2; half++) {
            const int ks = 2 * b + half;
            __half xh[4], xl[4];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const float x = qv[ks][i] * p.scale_log2;
                xh[i] = __float2half_rn(x);
                xl[i] = __float2half_rn(x - __half2float(xh[i]));
                sum += __half2float(xh[i]) + __half2float(xl[i]);
            }
            qb[ks][0] = pack_half2(xh[0], xh[1]);
            qb[ks][1] = pack_half2(xh[2], xh[3]);
            qb[ks][2] = pack_half2(xl[0], xl[1]);
            qb[ks][3] = pack_half2(xl[2], xl[3]);
        }
        // the four lanes of a head hold a quarter of the block each; the score accumulators of
        // lane (g, t) are heads 2t and 2t + 1 and start at -2^-17 * (sum over the block), which
        // takes the codes' offset of 128 out again (nibbles carry an offset of 8)
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        const float bias = -(kQ4 ? kCodeBias / 16.0f : kCodeBias) * sum;
        qbias[b][0] = __shfl_sync(0xffffffffu, bias, (2 * t) * 4);
        qbias[b][1] = __shfl_sync(0xffffffffu, bias, (2 * t + 1) * 4);
    }
    // (set-up wrote the barriers; the first tiles are on their way)
    __syncthreads();

    float acc[4][4];  // block `warp`: [byte i of the code word][c0..c3]
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int c = 0; c < 4; c++) acc[i][c] = 0.0f;
    float m_run = -INFINITY, l_run = 0.0f;  // meaningful in warp g' = head of the group

    bool landed = true;
    for (int tile = 0; tile < ntiles; tile++) {
        const int buf = tile % kStages;
        // the stage of tile + 2 was read last by tile - 1, which every warp has left
        if (tid == 0 && tile + 2 < ntiles) fetch(tile + 2);
        {
            const unsigned bar = bar_full + 8 * buf, parity = (unsigned)(tile / kStages) & 1u;
            unsigned spin = 0;
            while (!mbar_try_wait(bar, parity)) {
                if (++spin > kSpinLimit) {  // the copy never landed: flag it and carry on
                    landed = false;
                    break;
                }
            }
        }
        const int nvalid = min(kTile, hi - (lo + tile * kTile));
        unsigned char *const ktile_b = ktile_at(buf), *const vtile_b = vtile_at(buf);
        // (no barrier here: every thread has seen the copy land for itself)
        if (p.k_row != nullptr) {
            // Fused append: the row at the append position was copied as it was before this
            // step. Warp 0 (K) and warp 1 (V) quantise the new row into the tile, with the
            // encoder's own arithmetic, and store its bytes to the cache.
            const int prow = append_pos - (lo + tile * kTile);
            if (prow >= 0 && prow < nvalid) {
                if (warp < 2) {
                    const float *src = (warp == 0 ? p.k_row : p.v_row) + (size_t)slot * p.row_slot +
                                       (size_t)kvh * 256 + lane * 8;
                    unsigned char *row = (warp == 0 ? ktile_b : vtile_b) + prow * kSrcRow;
                    const float4 a = __ldg(reinterpret_cast<const float4 *>(src));
                    const float4 b = __ldg(reinterpret_cast<const float4 *>(src) + 1);
                    if constexpr (kQ4)
                        q4_put8(a, b, lane, row);
                    else
                        q8_put8(a, b, lane, row);
                    __syncwarp();
                    row_store((warp == 0 ? p.kw : p.vw) + head_byte + (size_t)append_pos * kSrcRow, row,
                              kSrcRow, lane, 32);
                }
                __syncthreads();
            }
        }
        if (nvalid < kTile) {
            // Rows past the split's end hold stale bytes; their V scales must read as zero.
            for (int i = tid; i < (kTile - nvalid) * (kSrcRow / 16); i += kThreads)
                reinterpret_cast<uint4 *>(vtile_b + nvalid * kSrcRow)[i] = make_uint4(0, 0, 0, 0);
        }

        // ---- (1) scores
        {
            float s[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            if constexpr (kQ4) {
                if (dh == 0) {
                    score_block_q4<0>(ktile_b, kg * 16, g, t, qb[0], qb[1], qbias[0], s);
                    score_block_q4<1>(ktile_b, kg * 16, g, t, qb[2], qb[3], qbias[1], s);
                    score_block_q4<2>(ktile_b, kg * 16, g, t, qb[4], qb[5], qbias[2], s);
                    score_block_q4<3>(ktile_b, kg * 16, g, t, qb[6], qb[7], qbias[3], s);
                } else {
                    score_block_q4<4>(ktile_b, kg * 16, g, t, qb[0], qb[1], qbias[0], s);
                    score_block_q4<5>(ktile_b, kg * 16, g, t, qb[2], qb[3], qbias[1], s);
                    score_block_q4<6>(ktile_b, kg * 16, g, t, qb[4], qb[5], qbias[2], s);
                    score_block_q4<7>(ktile_b, kg * 16, g, t, qb[6], qb[7], qbias[3], s);
                }
            } else if (dh == 0) {
                score_block<0>(ktile_b, kg * 16, g, t, qb[0], qb[1], qbias[0], s);
                score_block<1>(ktile_b, kg * 16, g, t, qb[2], qb[3], qbias[1], s);
                score_block<2>(ktile_b, kg * 16, g, t, qb[4], qb[5], qbias[2], s);
                score_block<3>(ktile_b, kg * 16, g, t, qb[6], qb[7], qbias[3], s);
            } else {
                score_block<4>(ktile_b, kg * 16, g, t, qb[0], qb[1], qbias[0], s);
                score_block<5>(ktile_b, kg * 16, g, t, qb[2], qb[3], qbias[1], s);
                score_block<6>(ktile_b, kg * 16, g, t, qb[4], qb[5], qbias[2], s);
                score_block<7>(ktile_b, kg * 16, g, t, qb[6], qb[7], qbias[3], s);
            }
            float *dst = ss + (dh * 8 + 2 * t) * kSsStride + kg * 16 + g;
            dst[0] = s[0];
            dst[kSsStride] = s[1];
            dst[8] = s[2];
            dst[kSsStride + 8] = s[3];
        }
        __syncthreads();

        // ---- (2) softmax: warp = head of the group, lane = keys 2*lane, 2*lane+1
        {
            const float2 a = *reinterpret_cast<const float2 *>(ss + warp * kSsStride + 2 * lane);
            const float2 b = *reinterpret_cast<const float2 *>(ss + (8 + warp) * kSsStride + 2 * lane);
            const float s0 = 2 * lane < nvalid ? (a.x + b.x) * kCodeUnit : -INFINITY;
            const float s1 = 2 * lane + 1 < nvalid ? (a.y + b.y) * kCodeUnit : -INFINITY;
            const float m_new = fmaxf(m_run, warp_max(fmaxf(s0, s1)));
            // m_new is -inf only while every key so far was masked: nothing to scale then.
            const float corr = (m_new == -INFINITY) ? 1.0f : exp2f(m_run - m_new);
            const float p0 = (s0 == -INFINITY) ? 0.0f : exp2f(s0 - m_new);
            const float p1 = (s1 == -INFINITY) ? 0.0f : exp2f(s1 - m_new);
            l_run = l_run * corr + warp_sum(p0 + p1);
            m_run = m_new;
            const float w0 = p0 * kPScale, w1 = p1 * kPScale;
            const __half h0 = __float2half_rn(w0), h1 = __float2half_rn(w1);
            const __half l0 = __float2half_rn(w0 - __half2float(h0));
            const __half l1 = __float2half_rn(w1 - __half2float(h1));
            *reinterpret_cast<unsigned *>(ph + warp * kPStride + 2 * lane) = pack_half2(h0, h1);
            *reinterpret_cast<unsigned *>(pl + warp * kPStride + 2 * lane) = pack_half2(l0, l1);
            if (lane == 0) corr_s[warp] = corr;
        }
        __syncthreads();

        // ---- (3) values: warp = block (32 dims), all 64 keys
        if constexpr (kQ4) {
            if (warp & 1)
                values_block_q4<true>(vtile_b, warp, g, t, ph, pl, corr_s[g], acc);
            else
                values_block_q4<false>(vtile_b, warp, g, t, ph, pl, corr_s[g], acc);
        } else if (warp & 1) {
            values_block<true>(vtile_b, warp, g, t, ph, pl, corr_s[g], acc);
        } else {
            values_block<false>(vtile_b, warp, g, t, ph, pl, corr_s[g], acc);
        }
        __syncthreads();  // tile buffers, ss and the weight tile are reused by the next tile
    }

    if (!landed && status) atomicCAS(status, 0, 21);

    // ---- partials. Output column n of MMA i is dim 32*blk + 4n + i; this thread holds
    // columns 2t, 2t+1, i.e. dims 32*blk + 8t + i and 32*blk + 8t + 4 + i of head g
    // (c0/c1: high-part row, c2/c3: low-part row).
    if (g < group) {
        const int h = kvh * group + g;
        float *pa = p.part_acc + (size_t)slot * p.acc_slot + ((size_t)h * p.splits + split) * 256 +
                    warp * 32 + 8 * t;
        const float inv = 1.0f / kPScale;
        *reinterpret_cast<float4 *>(pa) =
            make_float4((acc[0][0] + acc[0][2]) * inv, (acc[1][0] + acc[1][2]) * inv,
                        (acc[2][0] + acc[2][2]) * inv, (acc[3][0] + acc[3][2]) * inv);
        *reinterpret_cast<float4 *>(pa + 4) =
            make_float4((acc[0][1] + acc[0][3]) * inv, (acc[1][1] + acc[1][3]) * inv,
                        (acc[2][1] + acc[2][3]) * inv, (acc[3][1] + acc[3][3]) * inv);
    }
    if (warp < group && lane == 0) {
        const int h = kvh * group + warp;
        float *pm = p.part_ml + (size_t)slot * p.ml_slot + ((size_t)h * p.splits + split) * 2;
        pm[0] = m_run;
        pm[1] = l_run;
    }
    }   // ntiles > 0

    // ---- fold inside the split pass
    if (p.out == nullptr) return;
    const int runs = live_runs(p, slot, p.share_slots > 0 ? s_plan[3] : 0);
    if (split >= runs) return;   // a launched run past the live ones: its neutral partial is not read
    fold_tail(p, status, slot, kvh, split, runs, group, tid);
}

// ------------------------------------------------------------------------------------------
// The q8_0 body with the value side on the 5th-generation tensor cores (tcgen05.mma kind::i8,
// accumulators in TMEM). Scores, tiles, run plan, fused append and fold are those of
// attn_decode_kv_tc; what changes is phase (3):
//   * the V tile is brought in by 17 tensor (TMA) copies of {16 bytes, 64 rows}, one per
//     16-byte column chunk of the 272-byte rows, so it lands as [chunk][key][16 B]: exactly the
//     canonical MN-major operand of the MMA (8 keys x 16 bytes contiguous per core matrix).
//     The int8 codes are the A operand as they are: M = byte of the row (three M tiles of 128
//     cover the 272 bytes; the two scale bytes of each block are rows whose results are never
//     read), K = key. No conversion of a single code on the CUDA cores;
//   * the B operand is built per tile: column (block b, head h, digit) holds the weight
//     exp2(score - ref_h) * scale(key, b) as a 23-bit fixed-point number in three unsigned
//     bytes, taken straight out of the mantissa of weight * F + 2^23. A block's results only
//     need that block's columns, so an M tile multiplies a window of 32 .. 96 columns;
//   * products accumulate as int32 in TMEM (exact); per head the reference `ref_h` of the
//     exponentials and the unit of the value scales stay fixed while the running maximum stays
//     within 2^5.5 of it, so the accumulators are read out only when a reference moves (a few
//     times per run) and at the end: digits are combined and scaled in f32 there.
// Weights carry 17 bits below the reference (error 2^-18 of the largest weight), the int32
// sums are exact, scores are as before: results agree with the f32 definition to ~1e-6.
namespace i8 {

constexpr float kMagicLimit = 8388608.0f;
constexpr int kKStages = 2;                    // the K tile is free once its scores are out
constexpr int kVStages = 3;                    // the V tile until its MMAs have run
constexpr int kDigits = 3;
constexpr int kCols = 6 * kDigits;               // columns per block: 6 heads x 3 digits
constexpr int kBRows = 162;                      // 8 * 18 weight rows + what the last windows read past them;
                                                 // 162 * 16 B keeps the four key chunks on different banks
constexpr int kBChunk = kBRows * 16;             // bytes between 16-key chunks of the B operand
constexpr int kOffV = kKStages * kTileBytes;                // K ring first
constexpr int kOffB = kOffV + kVStages * kTileBytes;
constexpr int kOffSs = kOffB + 4 * kBChunk;                 // scores [2][8][kSsStride] f32
constexpr int kOffPw = kOffSs + 2 * 8 * kSsStride * 4;      // weights' exponentials [6][64] f32
constexpr int kOffDv = kOffPw + 6 * 64 * 4;                 // value scales [8][64] f32
constexpr int kOffMisc = kOffDv + 8 * 64 * 4;               // fscale[8] f32, dvmax bits, flush flag
constexpr int kOffRow = kOffMisc + 64;                      // one row image (fused append)
constexpr int kOffBar = kOffRow + 288;                      // K full [2], V full [3], MMA done
constexpr int kSmem = kOffBar + 64;
static_assert(2 * (kSmem + 1024) <= 227 * 1024, "two CTAs per SM");
// the M tile that starts at chunk 16 reads 8 chunks: 7 KB past the V stage, still inside the window
static_assert(kOffV + kVStages * kTileBytes + 7 * 1024 <= kSmem, "M tile 2 reads past the stage");
constexpr unsigned kTmemCols = 256;
// M tile mt covers row bytes [128 mt, 128 mt + 128) = blocks {0..3}, {3..7}, {7}: window of B rows
// [n0, n0 + N) and TMEM columns [tcol, tcol + N)
__device__ __forceinline__ int win_n0(int mt) { return mt == 0 ? 0 : (mt == 1 ? 48 : 120); }
__device__ __forceinline__ int win_n(int mt) { return mt == 0 ? 80 : (mt == 1 ? 96 : 32); }
__device__ __forceinline__ int win_tcol(int mt) { return mt == 0 ? 0 : (mt == 1 ? 80 : 176); }
constexpr float kHeadroom = 3.0f;                // log2 units: exponentials stay below 2^3 of the reference
constexpr float kDvSlack = 1.25f;                // the unit of the value scales: this much above the largest seen
constexpr float kFixedOne = 524288.0f;           // 2^19: fixed-point value of weight 1 at the unit scale
static_assert(8.0f * kFixedOne < kMagicLimit, "the largest weight (2^3 at the unit scale) must stay below 2^23");
constexpr float kMagic = 8388608.0f;             // 2^23: weight * F + 2^23 has the integer in its mantissa

__device__ __forceinline__ uint64_t desc_nosw(unsigned addr, unsigned lbo, unsigned sbo) {
    return (uint64_t)((addr & 0x3ffff) >> 4) | ((uint64_t)((lbo >> 4) & 0x3fff) << 16) |
           ((uint64_t)((sbo >> 4) & 0x3fff) << 32) | ((uint64_t)1 << 46);
}
// s32 accumulate, A = s8 MN-major, B = u8 K-major, M = 128
__device__ __forceinline__ unsigned idesc_i8(unsigned n) {
    return (2u << 4) | (1u << 7) | (0u << 10) | (1u << 15) | ((n >> 3) << 17) | ((128u >> 4) << 24);
}
__device__ __forceinline__ void mma_i8(unsigned d, uint64_t a, uint64_t b, unsigned idesc, unsigned accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void tmem_ld4(unsigned taddr, unsigned (&r)[4]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(taddr)
                 : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Adds what the accumulators of this thread's row byte hold to acc (f32), in `unit`s. The warp's
// 32 row bytes lie in at most two blocks, whose 36 columns are read with one address.
__device__ __forceinline__ void readout(unsigned tmem, int mt, int lane_base, int lane, float unit,
                                        float (&acc)[6]) {
    const int byte0 = 128 * mt + lane_base;
    const int blk_lo = byte0 / 34;
    const bool second = (byte0 + lane) / 34 != blk_lo;
    const unsigned taddr = tmem + ((unsigned)lane_base << 16) + win_tcol(mt) + kCols * blk_lo - win_n0(mt);
    unsigned r[32], r2[4];
    tmem_ld32(taddr, r);
    tmem_ld4(taddr + 32, r2);
#pragma unroll
    for (int h = 0; h < 6; h++) {
        int d[3];
#pragma unroll
        for (int j = 0; j < 3; j++) {
            const int lo = (int)r[3 * h + j];
            const int idx = kCols + 3 * h + j;   // the same column of the warp's second block
            const int hi = idx < 32 ? (int)r[idx] : (int)r2[idx - 32];
            d[j] = second ? hi : lo;
        }
        const float v = fmaf((float)d[2], 65536.0f, fmaf((float)d[1], 256.0f, (float)d[0]));
        acc[h] = fmaf(v, unit, acc[h]);
    }
}

__device__ __forceinline__ void tma_load_3d(unsigned dst, const CUtensorMap *map, int x, int y, int z,
                                            unsigned bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar)
        : "memory");
}

// vmap: the V cache as rows of 272 bytes. v3d != 0: a 3-D view {16 bytes, rows, 17 chunks} whose
// box {16, 64, 17} lands a whole tile in chunk order with one copy; else a 2-D view {272, rows}
// with box {16, 64}, one copy per chunk.
__global__ void __launch_bounds__(kThreads, 2)
attn_decode_kv_i8(const __grid_constant__ CUtensorMap vmap, int v3d, DecodeParams p, int *status) {
    extern __shared__ __align__(128) unsigned char smem_i8[];
    unsigned char *const smem = smem_i8;
    griddep_launch();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int group = p.n_heads / p.n_kv;
    const int kg = warp & 3, dh = warp >> 2;
    unsigned *tmem_slot = reinterpret_cast<unsigned *>(smem + kOffBar + 56);
    if (warp == 0) {
        // (nothing of memory is touched; a CTA of the grid before may still hold its columns)
        tmem_alloc<1>(smem_u32(tmem_slot), kTmemCols);
    }
    // Everything this kernel reads may come from the grids before it: nothing is read before this.
    griddep_wait();
    auto ktile_at = [&](int stage) { return smem + stage * kTileBytes; };   // kKStages of them
    auto vtile_at = [&](int stage) { return smem + kOffV + stage * kTileBytes; };
    unsigned char *bop = smem + kOffB;
    float *ss = reinterpret_cast<float *>(smem + kOffSs);
    float *pw = reinterpret_cast<float *>(smem + kOffPw);            // [6][64]
    float *sdv = reinterpret_cast<float *>(smem + kOffDv);           // [8][64]
    float *s_fscale = reinterpret_cast<float *>(smem + kOffMisc);    // [8]
    // per tile parity: the tile's largest value scale (f32 bits) and "a reference moved"
    unsigned *s_dvmax = reinterpret_cast<unsigned *>(smem + kOffMisc + 32);   // [2]
    int *s_flush = reinterpret_cast<int *>(smem + kOffMisc + 40);             // [2]
    unsigned char *rowbuf = smem + kOffRow;

    __shared__ int s_plan[4];   // slot (-1: none), kvh, split, quota
    const int grid_splits = (p.by_stride || p.run_cap <= 0) ? p.splits : min(p.splits, p.run_cap);
    int slot = blockIdx.y, kvh = blockIdx.x / grid_splits, split = blockIdx.x - kvh * grid_splits;
    if (p.share_slots > 0) {
        if (warp == 1) {
            const int quota = shared_quota_warp(p.len, p.len_stride, p.len_offset, p.n_slots, p.splits,
                                                p.share_slots, p.n_kv);
            const int b = blockIdx.x;
            int base = 0;
            if (lane == 0) {
                s_plan[0] = -1;
                s_plan[3] = quota;
            }
            __syncwarp();
            for (int s0 = 0; s0 < p.n_slots; s0 += 32) {
                const int s = s0 + lane;
                const int per = s < p.n_slots
                    ? shared_runs_of((p.len[s * p.len_stride + p.len_offset] + 63) >> 6, quota) : 0;
                const int runs = per * p.n_kv;
                int incl = runs;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const int up = __shfl_up_sync(0xffffffffu, incl, o);
                    if (lane >= o) incl += up;
                }
                const int first = base + incl - runs;
                if (runs > 0 && b >= first && b < first + runs) {
                    const int r = b - first;
                    s_plan[0] = s;
                    s_plan[1] = r / per;
                    s_plan[2] = r - (r / per) * per;
                }
                base += __shfl_sync(0xffffffffu, incl, 31);
            }
        }
        __syncthreads();
        slot = s_plan[0];
        kvh = s_plan[1];
        split = s_plan[2];
    }
    const bool idle = slot < 0;   // (the shared grid is one round of CTAs; the tail of it may be spare)

    // query values of this lane (see attn_decode_kv_tc), before anything that depends on the length
    float qv[8][4];
    if (!idle) {
        const float *qh = p.q + (size_t)slot * p.q_slot + (size_t)(kvh * group + g) * 256;
#pragma unroll
        for (int ks = 0; ks < 8; ks++) {
            const int blk = dh * 4 + (ks >> 1), j = (ks & 1) * 4 + t;
#pragma unroll
            for (int i = 0; i < 4; i += 2) {
                float2 x = make_float2(0.0f, 0.0f);
                if (g < group) x = *reinterpret_cast<const float2 *>(qh + k_word_dim(blk, j, i));
                qv[ks][i] = x.x;
                qv[ks][i + 1] = x.y;
            }
        }
    }
    int lo = 0, hi = 0;
    if (!idle) split_range(p, slot, split, p.share_slots > 0 ? s_plan[3] : 0, lo, hi);
    const int ntiles = (hi - lo + kTile - 1) / kTile;
    if (!idle && ntiles == 0) {
        // A split without rows: neutral partials (zero sum, -inf maximum), nothing else.
        for (int i = tid; i < group * 256; i += kThreads) {
            const int h = kvh * group + (i >> 8);
            p.part_acc[(size_t)slot * p.acc_slot + ((size_t)h * p.splits + split) * 256 + (i & 255)] = 0.0f;
        }
        if (tid < group) {
            float *pm = p.part_ml + (size_t)slot * p.ml_slot +
                        ((size_t)(kvh * group + tid) * p.splits + split) * 2;
            pm[0] = -INFINITY;
            pm[1] = 0.0f;
        }
    }

    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem = *tmem_slot;

    if (ntiles > 0) {
    const size_t head_byte = (size_t)slot * p.kv_slot_bytes + (size_t)kvh * p.stride * kRowBytes;
    const unsigned char *kbase = p.k + head_byte;
    // first row of this KV head in the V tensor of 272-byte rows
    const int vrow0 = (int)(((size_t)slot * p.kv_slot_bytes) / kRowBytes) + kvh * p.stride;
    int append_pos = -1;
    if (p.k_row != nullptr) {
        append_pos = p.len[slot * p.len_stride + p.len_offset - 1];
        if (split == 0 && kvh == 0 && tid == 0 &&
            append_pos != p.len[slot * p.len_stride + p.len_offset] - 1 && status)
            atomicCAS(status, 0, 22);
    }
    const unsigned bar_k = smem_u32(smem + kOffBar), bar_v = bar_k + 16, bar_mma = bar_k + 40;
    auto fetch_k = [&](int tile) {
        const int stage = tile % kKStages;
        const int r0 = lo + tile * kTile;
        const unsigned bytes = (unsigned)(min(kTile, hi - r0) * kRowBytes);
        fence_async_shared();
        mbar_arrive_expect_tx(bar_k + 8 * stage, bytes);
        bulk_load(smem_u32(ktile_at(stage)), kbase + (size_t)r0 * kRowBytes, bytes, bar_k + 8 * stage);
    };
    // 17 copies of {16 bytes, 64 rows}; rows past the run are other rows of the cache (or zeros
    // past its end): their weights are zero
    // (called by all lanes of one warp)
    auto fetch_v = [&](int tile) {
        const int stage = tile % kVStages;
        const unsigned dst = smem_u32(vtile_at(stage));
        fence_async_shared();
        if (lane == 0) mbar_arrive_expect_tx(bar_v + 8 * stage, (unsigned)kTileBytes);
        __syncwarp();
        if (v3d) {
            if (lane == 0) tma_load_3d(dst, &vmap, 0, vrow0 + lo + tile * kTile, 0, bar_v + 8 * stage);
        } else if (lane < 17) {
            tma_load_2d<1>(dst + lane * 1024, &vmap, 16 * lane, vrow0 + lo + tile * kTile, bar_v + 8 * stage);
        }
    };
    // warp 7 is the producer of both rings: two tiles are always on their way
    if (warp == 7) {
        if (lane == 0) {
#pragma unroll
            for (int s = 0; s < 6; s++) mbar_init(bar_k + 8 * s, 1);
            mbar_init_fence();
            s_dvmax[0] = s_dvmax[1] = 0u;
            s_flush[0] = s_flush[1] = 0;
            fetch_k(0);
            if (ntiles > 1) fetch_k(1);
        }
        __syncwarp();
        fetch_v(0);
        if (ntiles > 1) fetch_v(1);
    }

    unsigned qb[8][4];
    float qbias[4][2];
#pragma unroll
    for (int b = 0; b < 4; b++) {
        float sum = 0.0f;
#pragma unroll
        for (int half = 0; half < 2; half++) {
            const int ks = 2 * b + half;
            __half xh[4], xl[4];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const float x = qv[ks][i] * p.scale_log2;
                xh[i] = __float2half_rn(x);
                xl[i] = __float2half_rn(x - __half2float(xh[i]));
                sum += __half2float(xh[i]) + __half2float(xl[i]);
            }
            qb[ks][0] = pack_half2(xh[0], xh[1]);
            qb[ks][1] = pack_half2(xh[2], xh[3]);
            qb[ks][2] = pack_half2(xl[0], xl[1]);
            qb[ks][3] = pack_half2(xl[2], xl[3]);
        }
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        const float bias = -kCodeBias * sum;
        qbias[b][0] = __shfl_sync(0xffffffffu, bias, (2 * t) * 4);
        qbias[b][1] = __shfl_sync(0xffffffffu, bias, (2 * t + 1) * 4);
    }
    __syncthreads();

    // f32 accumulators of this thread's row byte, in units of 2^ref_h: warps 0..3 own bytes
    // 0..127 (M tile 0), warps 4..7 bytes 128..255 (M tile 1); warp 0 also bytes 256..271
    float acc[6] = {0, 0, 0, 0, 0, 0}, acc2[6] = {0, 0, 0, 0, 0, 0};
    const int mt = warp >> 2, lane_base = (warp & 3) * 32;
    float m_ref = -INFINITY, l_ref = 0.0f;   // meaningful in warp h = head of the group
    float dvref = 0.0f;                      // unit of the value scales (the same in every thread)
    bool fresh = true;                       // the accumulators in TMEM hold nothing yet
    bool mma_fresh = true;                   // ... as the MMAs of the tile before will find them
    // O += codes^T x weights of `tile`: three M tiles, two steps of 32 keys each (one thread)
    auto issue_mma = [&](int tile, bool overwrite) {
        tc_fence_after();
        const unsigned va = smem_u32(vtile_at(tile % kVStages)), ba = smem_u32(bop);
#pragma unroll
        for (int m = 0; m < 3; m++) {
            const unsigned idesc = idesc_i8((unsigned)win_n(m));
#pragma unroll
            for (int ks = 0; ks < 2; ks++)
                mma_i8(tmem + win_tcol(m), desc_nosw(va + m * 8 * 1024 + ks * 512, 128, 1024),
                       desc_nosw(ba + win_n0(m) * 16 + ks * 2 * kBChunk, kBChunk, 128), idesc,
                       (ks != 0 || !overwrite) ? 1u : 0u);
        }
        tc_commit<1>(bar_mma);
    };
    bool landed = true;
    auto wait_bar = [&](unsigned bar, unsigned parity) {
        unsigned spin = 0;
        while (!mbar_try_wait(bar, parity)) {
            if (++spin > kSpinLimit) {
                landed = false;
                break;
            }
        }
    };

    for (int tile = 0; tile < ntiles; tile++) {
        const int kbuf = tile % kKStages, vbuf = tile % kVStages;
        wait_bar(bar_k + 8 * kbuf, (unsigned)(tile / kKStages) & 1u);
        const int nvalid = min(kTile, hi - (lo + tile * kTile));
        unsigned char *const ktile_b = ktile_at(kbuf), *const vtile_b = vtile_at(vbuf);
        if (p.k_row != nullptr) {
            const int prow = append_pos - (lo + tile * kTile);
            if (prow >= 0 && prow < nvalid) {
                if (warp == 0) {
                    const float *src = p.k_row + (size_t)slot * p.row_slot + (size_t)kvh * 256 + lane * 8;
                    unsigned char *row = ktile_b + prow * kRowBytes;
                    q8_put8(__ldg(reinterpret_cast<const float4 *>(src)),
                            __ldg(reinterpret_cast<const float4 *>(src) + 1), lane, row);
                    __syncwarp();
                    row_store(p.kw + head_byte + (size_t)append_pos * kRowBytes, row, kRowBytes, lane, 32);
                } else if (warp == 1) {
                    // the V row: built as a row image, copied into the tile's chunk order and stored
                    wait_bar(bar_v + 8 * vbuf, (unsigned)(tile / kVStages) & 1u);
                    const float *src = p.v_row + (size_t)slot * p.row_slot + (size_t)kvh * 256 + lane * 8;
                    q8_put8(__ldg(reinterpret_cast<const float4 *>(src)),
                            __ldg(reinterpret_cast<const float4 *>(src) + 1), lane, rowbuf);
                    __syncwarp();
                    if (lane < 17)
                        *reinterpret_cast<uint4 *>(vtile_b + lane * 1024 + prow * 16) =
                            *reinterpret_cast<const uint4 *>(rowbuf + lane * 16);
                    row_store(p.vw + head_byte + (size_t)append_pos * kRowBytes, rowbuf, kRowBytes, lane, 32);
                }
                __syncthreads();
            }
        }

        // ---- (1) scores
        {
            float s[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            if (dh == 0) {
                score_block<0>(ktile_b, kg * 16, g, t, qb[0], qb[1], qbias[0], s);
                score_block<1>(ktile_b, kg * 16, g, t, qb[2], qb[3], qbias[1], s);
                score_block<2>(ktile_b, kg * 16, g, t, qb[4], qb[5], qbias[2], s);
                score_block<3>(ktile_b, kg * 16, g, t, qb[6], qb[7], qbias[3], s);
            } else {
                score_block<4>(ktile_b, kg * 16, g, t, qb[0], qb[1], qbias[0], s);
                score_block<5>(ktile_b, kg * 16, g, t, qb[2], qb[3], qbias[1], s);
                score_block<6>(ktile_b, kg * 16, g, t, qb[4], qb[5], qbias[2], s);
                score_block<7>(ktile_b, kg * 16, g, t, qb[6], qb[7], qbias[3], s);
            }
            float *dst = ss + (dh * 8 + 2 * t) * kSsStride + kg * 16 + g;
            dst[0] = s[0];
            dst[kSsStride] = s[1];
            dst[8] = s[2];
            dst[kSsStride + 8] = s[3];
        }
        __syncthreads();
        // the K stage is free again: tile + 2 goes there
        if (tid == 6 * 32 && tile + 2 < ntiles) fetch_k(tile + 2);
        // The weights of the tile before are complete in every warp (and their V tile landed: this
        // thread waited for it then): their MMAs run beside this tile's exponentials.
        if (tid == 7 * 32 && tile >= 1) issue_mma(tile - 1, mma_fresh);

        // ---- (2) exponentials (warp = head, lane = keys 2*lane, 2*lane + 1), and beside them the
        // value scales of the tile as f32 with their maximum (warps 6, 7: one key per lane)
        if (warp < group) {
            const float2 a = *reinterpret_cast<const float2 *>(ss + warp * kSsStride + 2 * lane);
            const float2 b = *reinterpret_cast<const float2 *>(ss + (8 + warp) * kSsStride + 2 * lane);
            const float s0 = 2 * lane < nvalid ? (a.x + b.x) * kCodeUnit : -INFINITY;
            const float s1 = 2 * lane + 1 < nvalid ? (a.y + b.y) * kCodeUnit : -INFINITY;
            const float tmax = warp_max(fmaxf(s0, s1));
            // the reference of this head's exponentials moves only when the tile's maximum leaves
            // the headroom above it (or at the first tile): the accumulators then restart
            const bool move = m_ref == -INFINITY || tmax > m_ref + kHeadroom;
            const float ref = move ? tmax : m_ref;
            const float fs = (m_ref == -INFINITY || !move) ? 1.0f : exp2f(m_ref - ref);
            l_ref *= fs;
            m_ref = ref;
            const float p0 = (s0 == -INFINITY) ? 0.0f : exp2f(s0 - m_ref);
            const float p1 = (s1 == -INFINITY) ? 0.0f : exp2f(s1 - m_ref);
            l_ref += warp_sum(p0 + p1);
            *reinterpret_cast<float2 *>(pw + warp * 64 + 2 * lane) = make_float2(p0, p1);
            if (lane == 0) {
                s_fscale[warp] = fs;
                if (move) s_flush[tile & 1] = 1;
            }
        } else if (warp >= 6) {
            wait_bar(bar_v + 8 * vbuf, (unsigned)(tile / kVStages) & 1u);
            const int k = (warp - 6) * 32 + lane;
            float mx = 0.0f;
#pragma unroll
            for (int b = 0; b < 8; b++) {
                const int at = b * kQ8BlockBytes;   // byte of the row where block b's scale sits
                const unsigned short bits =
                    *reinterpret_cast<const unsigned short *>(vtile_b + (at >> 4) * 1024 + k * 16 + (at & 15));
                float d = 0.0f;
                if (k < nvalid) {
                    // q8_0 scales are amax / 127 >= 0; anything else (negative, inf, NaN) is not a
                    // cache this body can weigh: flagged, read as zero
                    if (bits >= 0x7c00u) {
                        if (status) atomicCAS(status, 0, 23);
                    } else {
                        d = half_bits_to_float(bits);
                    }
                }
                sdv[b * 64 + k] = d;
                mx = fmaxf(mx, d);
            }
            mx = warp_max(mx);
            if (lane == 0) atomicMax(s_dvmax + (tile & 1), __float_as_uint(mx));
        }
        __syncthreads();

        // ---- (3) a reference moved: the accumulators leave TMEM (old units), then restart
        const float dvmax = __uint_as_float(s_dvmax[tile & 1]);
        const bool flush = s_flush[tile & 1] != 0 || dvmax > dvref;
        if (tid == 0) {
            // (the other parity was read by every thread a tile ago and is written a tile from now)
            s_dvmax[(tile + 1) & 1] = 0u;
            s_flush[(tile + 1) & 1] = 0;
        }
        // the MMAs of the tile before are done: their B operand may be rewritten, TMEM read
        if (tile >= 1) wait_bar(bar_mma, (unsigned)(tile - 1) & 1u);
        tc_fence_after();
        // ... and the V stage they read takes tile + 2
        if (warp == 7 && tile + 2 < ntiles) fetch_v(tile + 2);
        if (flush) {
            if (!fresh) {
                const float unit = dvref / kFixedOne;
                readout(tmem, mt, lane_base, lane, unit, acc);
                if (warp == 0) readout(tmem, 2, 0, lane, unit, acc2);
            }
#pragma unroll
            for (int h = 0; h < 6; h++) {
                const float fs = h < group ? s_fscale[h] : 1.0f;
                acc[h] *= fs;
                acc2[h] *= fs;
            }
            if (dvmax > dvref) dvref = kDvSlack * dvmax;
            fresh = true;
            tc_fence_before();
        }

        // ---- (4) weights: warp = block, lane = (three heads, four keys)
        {
            const int kq = lane & 15, hh = lane >> 4;
            const float f = dvref > 0.0f ? kFixedOne / dvref : 0.0f;
            const float4 dv = *reinterpret_cast<const float4 *>(sdv + warp * 64 + 4 * kq);
            const float d0 = dv.x * f, d1 = dv.y * f, d2 = dv.z * f, d3 = dv.w * f;
            unsigned char *dst = bop + (kq >> 2) * kBChunk + (kq & 3) * 4;
#pragma unroll
            for (int j = 0; j < 3; j++) {
                const int h = 3 * hh + j;
                const float4 pe = *reinterpret_cast<const float4 *>(pw + h * 64 + 4 * kq);
                const unsigned w0 = __float_as_uint(fmaf(pe.x, d0, kMagic));
                const unsigned w1 = __float_as_uint(fmaf(pe.y, d1, kMagic));
                const unsigned w2 = __float_as_uint(fmaf(pe.z, d2, kMagic));
                const unsigned w3 = __float_as_uint(fmaf(pe.w, d3, kMagic));
                // digit j of the four keys = byte j of the four mantissas
                const unsigned lo01 = __byte_perm(w0, w1, 0x5140);   // [w0.b0 w1.b0 w0.b1 w1.b1]
                const unsigned lo23 = __byte_perm(w2, w3, 0x5140);
                const unsigned hi01 = __byte_perm(w0, w1, 0x0062);   // [w0.b2 w1.b2 . .]
                const unsigned hi23 = __byte_perm(w2, w3, 0x0062);
                const int n = kCols * warp + kDigits * h;
                *reinterpret_cast<unsigned *>(dst + (n + 0) * 16) = __byte_perm(lo01, lo23, 0x5410);
                *reinterpret_cast<unsigned *>(dst + (n + 1) * 16) = __byte_perm(lo01, lo23, 0x7632);
                *reinterpret_cast<unsigned *>(dst + (n + 2) * 16) = __byte_perm(hi01, hi23, 0x5410);
            }
        }
        // (the MMAs of this tile are issued after the next barrier, beside the next tile's phase 2)
        fence_async_shared();
        tc_fence_before();
        mma_fresh = fresh;
        fresh = false;
    }

    // ---- the end of the run: the last tile's MMAs, the last accumulators, then the partials
    __syncthreads();
    if (tid == 7 * 32) issue_mma(ntiles - 1, mma_fresh);
    wait_bar(bar_mma, (unsigned)(ntiles - 1) & 1u);
    tc_fence_after();
    {
        const float unit = dvref / kFixedOne;
        readout(tmem, mt, lane_base, lane, unit, acc);
        if (warp == 0) readout(tmem, 2, 0, lane, unit, acc2);
    }
    if (!landed && status) atomicCAS(status, 0, 21);
    {
        // row byte -> head dim: byte 34 b + 2 + i is dim 32 b + i; the two scale bytes hold nothing
        const int byte = 128 * mt + lane_base + lane, blk = byte / 34, i = byte - 34 * blk - 2;
        if (i >= 0) {
#pragma unroll
            for (int h = 0; h < 6; h++)
                if (h < group)
                    p.part_acc[(size_t)slot * p.acc_slot + ((size_t)(kvh * group + h) * p.splits + split) * 256 +
                               32 * blk + i] = acc[h];
        }
        if (warp == 0 && lane < 16) {
            // bytes 256..271 are codes 16..31 of block 7
#pragma unroll
            for (int h = 0; h < 6; h++)
                if (h < group)
                    p.part_acc[(size_t)slot * p.acc_slot + ((size_t)(kvh * group + h) * p.splits + split) * 256 +
                               240 + lane] = acc2[h];
        }
    }
    if (warp < group && lane == 0) {
        float *pm = p.part_ml + (size_t)slot * p.ml_slot + ((size_t)(kvh * group + warp) * p.splits + split) * 2;
        pm[0] = m_ref;
        pm[1] = l_ref;
    }
    }   // ntiles > 0

    // every access to TMEM is over in every warp before its columns go back
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        tmem_dealloc<1>(tmem, kTmemCols);
    }
    if (idle || p.out == nullptr) return;
    const int runs = live_runs(p, slot, p.share_slots > 0 ? s_plan[3] : 0);
    if (split >= runs) return;
    fold_tail(p, status, slot, kvh, split, runs, group, tid);
}

}  // namespace i8

// Stand-alone launch of the same fold: grid (n_kv, slots), 8 warps = the heads of the group.
__global__ void __launch_bounds__(kThreads) attn_decode_fold_tree(DecodeParams p, int *status) {
    griddep_launch();
    griddep_wait();
    __shared__ int s_quota;
    const int kvh = blockIdx.x, slot = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int group = p.n_heads / p.n_kv;
    if (p.share_slots > 0) {
        if (warp == 0) {
            const int q = shared_quota_warp(p.len, p.len_stride, p.len_offset, p.n_slots, p.splits,
                                            p.share_slots, p.n_kv);
            if (lane == 0) s_quota = q;
        }
        __syncthreads();
    }
    const int runs = live_runs(p, slot, p.share_slots > 0 ? s_quota : 0);
    const int gsize = fold_group_of(runs);
    const int ngroups = (runs + gsize - 1) / gsize;
    FoldAcc f;
    if (warp < group) {
        const int h = kvh * group + warp;
        float *pa = p.part_acc + (size_t)slot * p.acc_slot + (size_t)h * p.splits * 256;
        float *ml = p.part_ml + (size_t)slot * p.ml_slot + (size_t)h * p.splits * 2;
        for (int g = 0; g < ngroups; g++) {
            f = fold_warp(pa, ml, g * gsize, 1, min(gsize, runs - g * gsize), lane);
            if (ngroups > 1) fold_store_partial(pa, ml, g * gsize, f, lane);
        }
        if (ngroups > 1) {
            __threadfence();
            __syncwarp();
            f = fold_warp(pa, ml, 0, gsize, ngroups, lane);
        }
    }
    fold_finish(p, status, slot, kvh, group, f);
}

}  // namespace

namespace {

// Per-device set-up of the two kernels (dynamic shared memory limit, status word), done once.
int *decode_tc_setup(int *rc) {
    static std::mutex mu;
    static int *status_word[64] = {};   // nullptr = device not set up yet
    *rc = 0;
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    std::lock_guard<std::mutex> lock(mu);
    if (status_word[dev] == nullptr) {
        cudaError_t e = cudaFuncSetAttribute(attn_decode_kv_tc<false>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(attn_decode_kv_tc<true>,
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
        if (e != cudaSuccess) {
            *rc = (int)e;
            return nullptr;
        }
        status_word[dev] = device_status_word();
        if (status_word[dev] == nullptr) *rc = launch_status();
    }
    return status_word[dev];
}

std::atomic<int> g_two_launch_fold{0};
std::atomic<int> g_decode_body{1};   // 1: values on mma.sync, 2: values on tcgen05 kind::i8

int i8_setup() {
    static std::mutex mu;
    static bool done[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    std::lock_guard<std::mutex> lock(mu);
    if (!done[dev]) {
        const cudaError_t e = cudaFuncSetAttribute(i8::attn_decode_kv_i8,
                                                   cudaFuncAttributeMaxDynamicSharedMemorySize, i8::kSmem);
        if (e != cudaSuccess) return (int)e;
        done[dev] = true;
    }
    return 0;
}

}  // namespace

void decode_set_two_launch_fold(int on) { g_two_launch_fold.store(on ? 1 : 0); }
void decode_set_body(int body) { g_decode_body.store(body); }

// Which arrival-counter region a launch on `stream` uses. Two launches may share a region
// only if they cannot overlap on the device, so the key is what serialises launches: the
// stream (by its process-unique id), and under stream capture also the capture sequence (two
// graphs captured from one stream may later run side by side; capture ids start at 1, so a
// captured launch never shares a key with an eager one). A key keeps its region for
// the life of the process; when the regions run out the caller takes the two-launch form.
int decode_arrive_region(cudaStream_t stream, long long counters) {
    if (counters > kArriveRegionInts || g_two_launch_fold.load()) return -1;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return -1;
    unsigned long long sid = 0, cap = 0;
    cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
    if (cudaStreamGetCaptureInfo(stream, &st, &cap) != cudaSuccess) {
        cudaGetLastError();
        return -1;
    }
    if (st == cudaStreamCaptureStatusActive) {
        // (only capture-safe calls here) the streams of one capture are all alive, so their
        // handles tell them apart
        sid = (unsigned long long)reinterpret_cast<uintptr_t>(stream);
    } else {
        cap = 0;
        if (cudaStreamGetId(stream, &sid) != cudaSuccess) {
            cudaGetLastError();
            return -1;
        }
    }
    static std::mutex mu;
    static std::map<std::tuple<int, unsigned long long, unsigned long long>, int> table;
    static int next_free[64] = {};
    if (dev < 0 || dev >= 64) return -1;
    std::lock_guard<std::mutex> lock(mu);
    const auto key = std::make_tuple(dev, cap, sid);
    auto it = table.find(key);
    if (it != table.end()) return it->second;
    if (next_free[dev] >= kArriveRegions) return -1;
    const int region = next_free[dev]++;
    table.emplace(key, region);
    return region;
}

int launch_decode_fold_tree(cudaStream_t stream, const DecodeParams &p, int slots) {
    int rc = 0;
    int *status = decode_tc_setup(&rc);
    if (!status) return rc;
    DecodeParams q = p;
    q.n_slots = slots;
    return launch_pdl(attn_decode_fold_tree, dim3(q.n_kv, slots), dim3(kThreads), 0, stream, 1, q, status);
}

// Split pass; with p.out set also the fold: inside the same launch when an arrival-counter
// region is to be had, as a second launch otherwise.
int launch_decode_tc(cudaStream_t stream, const DecodeParams &p, int slots) {
    int rc = 0;
    int *status = decode_tc_setup(&rc);
    if (!status) return rc;
    dim3 grid(p.n_kv * p.splits, slots);
    DecodeParams q = p;
    q.n_slots = slots;
    if (q.share_slots > 0)
        grid = dim3(q.share_slots, 1);
    else if (!q.by_stride && q.run_cap > 0 && q.run_cap < q.splits)
        grid = dim3(q.n_kv * q.run_cap, slots);
    // The body with the value side on tcgen05 (int8 operands): q8_0, a GQA group of at most 6,
    // slots a whole number of 272-byte rows apart.
    // (selector 7 asks for the mma.sync values, selector 8 for the tcgen05 values; otherwise the
    // process-wide choice of hipml_set_decode_body, whose default is the faster of the two)
    const int want = q.legacy_body == 1 ? 1 : (q.legacy_body == 2 ? 2 : g_decode_body.load());
    const bool i8_body = want == 2 && !q.q4 && q.n_heads / q.n_kv <= 6 && q.kv_slot_bytes % kRowBytes == 0;
    CUtensorMap vmap;
    int v3d = 0;
    if (i8_body) {
        if (int e = i8_setup()) return e;
        EncodeTiledFn fn = encode_tiled_fn();
        if (!fn) return fail(HIPML_ERR_INVALID_ARGUMENT, "cuTensorMapEncodeTiled is not available");
        const cuuint64_t rows = (cuuint64_t)(slots > 1 ? (slots - 1) * (q.kv_slot_bytes / kRowBytes) : 0) +
                                (cuuint64_t)q.n_kv * q.stride;
        // the tile in chunk order with one copy: {16 bytes, rows (272 apart), 17 chunks (16 apart)}
        const cuuint64_t dims3[3] = {16, rows, 17};
        const cuuint64_t strides3[2] = {(cuuint64_t)kRowBytes, 16};
        const cuuint32_t box3[3] = {16, (cuuint32_t)kTile, 17};
        const cuuint32_t elem3[3] = {1, 1, 1};
        CUresult r = fn(&vmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<unsigned char *>(q.v), dims3,
                        strides3, box3, elem3, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        v3d = r == CUDA_SUCCESS;
        static const bool verbose = getenv("HIPML_VERBOSE") != nullptr;
        if (verbose)
            fprintf(stderr, "hipml: decode V tiles land with %s\n",
                    v3d ? "one 3-D tensor copy" : "17 2-D tensor copies (3-D view refused)");
        if (!v3d) {
            // the driver refuses the overlapping view: one copy per chunk from the plain 2-D view
            const cuuint64_t dims[2] = {(cuuint64_t)kRowBytes, rows};
            const cuuint64_t strides[1] = {(cuuint64_t)kRowBytes};
            const cuuint32_t box[2] = {16, (cuuint32_t)kTile};
            const cuuint32_t elem[2] = {1, 1};
            r = fn(&vmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<unsigned char *>(q.v), dims, strides,
                   box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        }
        if (r != CUDA_SUCCESS)
            return fail(HIPML_ERR_INVALID_ARGUMENT, "cuTensorMapEncodeTiled (V cache) failed: %d", (int)r);
    }
    bool second_launch = false;
    if (q.out != nullptr) {
        // most runs a (slot, KV head) can have under the plan in force
        int bound = q.splits;
        if (q.share_slots > 0) bound = min(bound, max(q.share_slots / q.n_kv, 1));
        else if (!q.by_stride && q.run_cap > 0) bound = min(bound, q.run_cap);
        q.arrive_stride = 1 + (bound + kFoldGroup - 1) / kFoldGroup;
        q.arrive_region = decode_arrive_region(stream, (long long)slots * q.n_kv * q.arrive_stride);
        if (q.arrive_region < 0) {
            second_launch = true;
            q.out = nullptr;
        }
    }
    if (i8_body)
        rc = launch_pdl(i8::attn_decode_kv_i8, grid, dim3(kThreads), (size_t)i8::kSmem, stream, 1, vmap, v3d, q,
                        status);
    else
        rc = q.q4 ? launch_pdl(attn_decode_kv_tc<true>, grid, dim3(kThreads), (size_t)kSmemBytes, stream, 1,
                               q, status)
                  : launch_pdl(attn_decode_kv_tc<false>, grid, dim3(kThreads), (size_t)kSmemBytes, stream, 1,
                               q, status);
    if (rc != 0 || !second_launch) return rc;
    q.out = p.out;
    return launch_pdl(attn_decode_fold_tree, dim3(q.n_kv, slots), dim3(kThreads), 0, stream, 1, q, status);
}

}  // namespace hipml
