// Causal chunk (prefill) attention on the 5th-generation tensor cores:
// tcgen05.mma with TMEM accumulators, operand tiles brought in by TMA.
//
// CPU definition: crates/hipml-core/src/attention.rs:56-102 applied per query row with
// seq = pos0 + t + 1. Kernels replaced: crates/hipml-kernels/kernels/attn_chunk_wmma.hip:187-399
// (one pass) and attn_chunk_full.hip:134-336 (key-split partials).
//
// Two launches per call.
//
// 1. attn_chunk_stage: converts the visible cache rows (f32 or q8_0) into the operand image
//    the tensor cores read: K as f16 [kv head][key][256] and V transposed as f16
//    [kv head][256][key], each as a high plane and a low plane (x = hi + lo, |lo| <= ulp(hi)/2).
//    A dequantised q8 value (f16 scale * int8 code) has at most 18 significant bits, so
//    hi + lo holds it exactly. Keys are padded with zeros to a multiple of 128. This pass
//    moves ~5 bytes per cache element against ~1.5e5 tensor FLOP per element of the chunk's
//    attention, i.e. about 1.5% of the call.
//
// 2. attn_chunk_tc: one CTA per (query tile, KV head[, key slice]). A query tile stacks the
//    GQA group along M: row r = query (r / group) of the tile, head (r % group) of the
//    group, 128 rows = 21 queries x 6 heads on the shipped shape, so one staged K/V tile
//    feeds all six heads. Per 128-key step:
//        S = Q K^T           tcgen05.mma  M=128 N=128 K=256, Q (A) and K (B) from shared memory
//        P = exp2(S - m)     eight softmax warps, two threads per TMEM lane (row), P written
//                            back over S in TMEM as f16 high/low pairs
//        O += P V            tcgen05.mma  M=128 N=2x128 K=128, P (A) from TMEM, V^T (B) from
//                            shared memory
//    Q stays resident in shared memory (128 KB as hi/lo f16, 128B-swizzled K-major); K and
//    V^T chunks of 32 KB (hi + lo tile of 128 rows x 64 elements) stream through a 3-stage
//    TMA ring. TMEM: O 256 columns + two S/P buffers of 128 columns, so QK^T of step i+1
//    overlaps the softmax of step i. Precision mode 0 issues three MMAs per product
//    (hi*hi + lo*hi + hi*lo) into the same accumulator, which brings the result within
//    ~1e-5 of the f32 definition; mode 1 issues hi*hi only (the reference kernel's own
//    single-pass f16 precision).
//
//
//    The default form runs CTA pairs (thread-block clusters of two, tcgen05 cta_group::2):
//    the two CTAs of a pair own consecutive query tiles of one KV head and walk the same key
//    tiles; one MMA of M = 256 spans both (each CTA's 128 rows accumulate in its own TMEM) and
//    takes half of its B operand from each CTA's shared memory, so each CTA loads only half of
//    every K tile (64 of the 128 keys) and half of every V^T tile (128 of the 256 dims). That
//    halves the bytes each SM pulls from L2 per FLOP and doubles the time one ring slot
//    lasts. The leader CTA's MMA thread issues for the pair; completion is signalled to both
//    CTAs' barriers (tcgen05.commit with a CTA mask), the peer's TMA loads complete on the
//    leader's barriers, and the peer's softmax warps arrive on the leader's barrier when
//    their P is written. Every load is an ordinary one-destination TMA copy into the issuing
//    CTA's own shared memory. The single-CTA form (M = 128) is kept for A/B.
//
// Roles: warps 0-7 softmax/epilogue (two threads per row: TMEM lane = row, each owns half of
// the score and output columns), warp 8 lane 0 TMA producer, warp 9 lane 0 MMA issuer (of
// the leader CTA in the pair form).
// Every mbarrier wait is bounded: when a wait runs out the thread
// records a code in the device status word, raises a CTA-wide abort flag that every other
// wait observes, and the CTA falls through to its teardown (TMEM is always released).
#include <cuda.h>

#include "params.cuh"
#include "q8_pack.cuh"
#include "sm100_ptx.cuh"

namespace hipml {

struct ChunkTcParams {
    const float *q;
    float *out;        // [tokens][n_heads*256], splits < 2
    float *part_acc;   // splits >= 2
    float *part_ml;
    int *status;
    int n_heads, n_kv, group;
    int pos0, tokens;
    int lpad;          // staged keys per head (multiple of 128)
    int qtile;         // queries per CTA = 128 / group
    float scale_log2;
    int splits, qslots;
    int single_pass;   // 1: hi*hi only
    const float *gate; // optional [tokens][n_heads*256]: out *= sigmoid(gate) (one-pass form only)
};

namespace {

constexpr int kD = 256;
constexpr int kKeyTile = 128;
constexpr int kStages = 3;
constexpr int kTileBytes = 128 * 128;            // 128 rows x 64 f16, swizzled
constexpr int kStageBytes = 2 * kTileBytes;      // hi + lo
constexpr int kQBytes = 8 * kTileBytes;          // 4 dim-chunks x (hi, lo)
constexpr int kTcThreads = 320;   // 8 softmax warps, TMA producer warp, MMA warp
constexpr int kXchBytes = 2 * 256 * 4;   // the two halves of a row meet here (double-buffered)
constexpr int kSmemNeed = kQBytes + kStages * kStageBytes + 256 /*barriers*/ + kXchBytes;
constexpr int kSmemBytes = 232448;        // everything an SM offers: kSmemNeed + 768 B of alignment slack
constexpr unsigned kSpinLimit = 1u << 22;        // polls per wait before giving up
constexpr float kRescaleThreshold = 8.0f;        // log2 units: P stays <= 256
// The tensor cores add into the f32 accumulators with less than f32 rounding: measured against
// the f32 definition, the relative-L2 error of O grows by ~3.5e-9 per key of an unbroken
// accumulation chain (3.4e-5 at 10,000 keys, 3.5e-4 at 100,000). Every kFlushTiles key tiles
// the softmax warps therefore move O out of TMEM into the output rows in memory (added there
// in f32 by the CUDA cores) and the next PV product starts a fresh accumulator, which bounds
// the chain at 8,192 keys whatever the depth. Rows that see at most 8,192 keys never flush.
constexpr int kFlushTiles = 64;

// ------------------------------------------------------------------ PTX helpers

using namespace ptx;

// Bounded wait. Returns false when the wait ran out (status word set, abort raised) or
// another thread of the CTA aborted.
// `peer_abort` is the shared::cluster address of the other CTA's abort flag (0: no peer).
__device__ __forceinline__ bool mbar_wait(unsigned bar, unsigned parity, volatile int *abort_flag,
                                          unsigned peer_abort, int *status, int code) {
    for (unsigned i = 0; i < kSpinLimit; i++) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 255) == 255 && *abort_flag) return false;
        if (i > 4096) __nanosleep(64);
    }
    atomicCAS(status, 0, code);
    *abort_flag = 1;
    if (peer_abort)
        asm volatile("st.relaxed.cluster.shared::cluster.u32 [%0], %1;" ::"r"(peer_abort), "r"(1)
                     : "memory");
    __threadfence_block();
    return false;
}

// ------------------------------------------------------------------ staging

struct StageParams {
    const void *k;
    const void *v;
    __half *k_hi, *k_lo;    // [n_kv][lpad][256]
    __half *vt_hi, *vt_lo;  // [n_kv][256][lpad]
    int n_kv, n_keys, lpad, kv_dtype, stride;
    int tile0;              // first 64-key tile this launch writes
};

__device__ __forceinline__ void split_half(float x, __half &hi, __half &lo) {
    hi = __float2half_rn(x);
    lo = __float2half_rn(x - __half2float(hi));
}
// The same for two values at once, as packed pairs {a in the low half, b in the high half}:
// one two-way conversion each way instead of two scalar ones.
__device__ __forceinline__ void split_half2(float a, float b, unsigned &hi, unsigned &lo) {
    const __half2 h = __floats2half2_rn(a, b);
    const float2 f = __half22float2(h);
    const __half2 l = __floats2half2_rn(a - f.x, b - f.y);
    hi = *reinterpret_cast<const unsigned *>(&h);
    lo = *reinterpret_cast<const unsigned *>(&l);
}

// Dequantised (or copied) values of 8 consecutive dims of one cache row; zeros past n_keys.
__device__ __forceinline__ void stage_fetch(const StageParams &p, const void *cache, int kvh,
                                            int key, int d0, float (&x)[8]) {
    if (key >= p.n_keys) {
#pragma unroll
        for (int j = 0; j < 8; j++) x[j] = 0.0f;
        return;
    }
    if (p.kv_dtype == 0) {
        const float4 *r = reinterpret_cast<const float4 *>(
            (const float *)cache + (size_t)key * (p.n_kv * kD) + kvh * kD + d0);
        const float4 a = r[0], b = r[1];
        x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w;
        x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
    } else if (p.kv_dtype == 2) {
        // q4_0: dims 8*sub .. 8*sub+7 of the block are the low (sub < 2) or high nibbles of
        // bytes 8*(sub & 1) .. +7
        const int blk = d0 >> 5, sub = (d0 >> 3) & 3;
        const unsigned char *b = (const unsigned char *)cache +
                                 q4_row_offset(kvh, p.stride, key, kD) + (size_t)blk * kQ4BlockBytes;
        const float d = half_bits_to_float(*(const unsigned short *)b);
        const unsigned short *c = (const unsigned short *)(b + 2 + (sub & 1) * 8);
        const int shift = (sub >> 1) * 4;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const unsigned short w = c[j];
            x[2 * j] = d * ((float)((w >> shift) & 0xf) - 8.0f);
            x[2 * j + 1] = d * ((float)((w >> (8 + shift)) & 0xf) - 8.0f);
        }
    } else {
        const int blk = d0 >> 5, sub = (d0 >> 3) & 3;
        const unsigned char *b = (const unsigned char *)cache +
                                 q8_row_offset(kvh, p.stride, key, kD) + (size_t)blk * kQ8BlockBytes;
        const float d = half_bits_to_float(*(const unsigned short *)b);
        const unsigned short *c = (const unsigned short *)(b + 2 + sub * 8);
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const unsigned short w = c[j];
            x[2 * j] = d * (float)(signed char)(w & 0xff);
            x[2 * j + 1] = d * (float)(signed char)(w >> 8);
        }
    }
}

__device__ __forceinline__ void stage_store8(__half *hi, __half *lo, size_t at, const float (&x)[8]) {
    __half h[8], l[8];
#pragma unroll
    for (int j = 0; j < 8; j++) split_half(x[j], h[j], l[j]);
    *reinterpret_cast<uint4 *>(hi + at) =
        make_uint4(pack2(h[0], h[1]), pack2(h[2], h[3]), pack2(h[4], h[5]), pack2(h[6], h[7]));
    *reinterpret_cast<uint4 *>(lo + at) =
        make_uint4(pack2(l[0], l[1]), pack2(l[2], l[3]), pack2(l[4], l[5]), pack2(l[6], l[7]));
}

// grid (tiles, n_kv, 3), block 256: 64 keys of one KV head; z = 0 stages K, z = 1, 2 the two
// 128-dim halves of V (three times the CTAs of a fused pass: the chunk's 2048 new keys
// would otherwise fill less than one wave of the device).
__global__ void __launch_bounds__(256) attn_chunk_stage(StageParams p) {
    __shared__ float vs[64][129];
    griddep_launch();
    griddep_wait();
    const int kvh = blockIdx.y, key0 = (p.tile0 + blockIdx.x) * 64;
    const int tid = threadIdx.x;
    if (blockIdx.z == 0) {
        // K: row-major copy. Thread -> dims [8*(tid%32), +8) of keys tid/32 + 8*i.
#pragma unroll 4
        for (int i = 0; i < 8; i++) {
            const int key = key0 + (tid >> 5) + 8 * i, d0 = (tid & 31) * 8;
            float x[8];
            stage_fetch(p, p.k, kvh, key, d0, x);
            stage_store8(p.k_hi, p.k_lo, ((size_t)kvh * p.lpad + key) * kD + d0, x);
        }
        return;
    }
    // V: transposed through shared memory, 128 dims per CTA.
    {
        const int dh = blockIdx.z - 1;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int kl = (tid >> 4) + 16 * i, d0 = (tid & 15) * 8;
            float x[8];
            stage_fetch(p, p.v, kvh, key0 + kl, dh * 128 + d0, x);
#pragma unroll
            for (int j = 0; j < 8; j++) vs[kl][d0 + j] = x[j];
        }
        __syncthreads();
        // Eight lanes write the 64 keys (128 contiguous bytes) of one dim: whole sectors.
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int item = tid + 256 * i, kb = (item & 7) * 8, d = item >> 3;
            float x[8];
#pragma unroll
            for (int j = 0; j < 8; j++) x[j] = vs[kb + j][d];
            stage_store8(p.vt_hi, p.vt_lo, ((size_t)kvh * kD + dh * 128 + d) * p.lpad + key0 + kb, x);
        }
    }
}

// ------------------------------------------------------------------ main kernel

// kCtas = 1: one CTA per query tile. kCtas = 2: launched as clusters of two along x; the
// K maps then have 64-key boxes (a CTA loads its half of the keys of a tile).
template <int kCtas>
__global__ void __launch_bounds__(kTcThreads, 1)
attn_chunk_tc(const __grid_constant__ CUtensorMap map_k_hi, const __grid_constant__ CUtensorMap map_k_lo,
              const __grid_constant__ CUtensorMap map_vt_hi,
              const __grid_constant__ CUtensorMap map_vt_lo, ChunkTcParams p) {
    extern __shared__ unsigned char smem_raw[];
    griddep_launch();
    unsigned char *smem =
        reinterpret_cast<unsigned char *>((reinterpret_cast<size_t>(smem_raw) + 1023) & ~(size_t)1023);
    if ((size_t)(smem - smem_raw) + kSmemNeed > (size_t)kSmemBytes) {
        // The dynamic window starts further from a 1 KB boundary than the slack covers.
        if (threadIdx.x == 0) atomicCAS(p.status, 0, 9);
        return;
    }
    unsigned char *q_smem = smem;                       // 8 tiles: hi chunks 0..3, lo chunks 0..3
    unsigned char *ring = smem + kQBytes;               // kStages x (hi tile, lo tile)
    uint64_t *bars = reinterpret_cast<uint64_t *>(ring + kStages * kStageBytes);
    // bars: full[3], empty[3], s_ready[2], p_ready[2], o_done[2], halves_met[2]
    volatile int *abort_flag = reinterpret_cast<volatile int *>(bars + 14);
    unsigned *tmem_slot = reinterpret_cast<unsigned *>(bars + 15);
    float *xch = reinterpret_cast<float *>(bars + 32);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // The launch order is heaviest first: x = 0 holds the last query tiles, which walk the
    // most keys, so the tail of the grid is made of the short tiles.
    const unsigned rank = kCtas == 2 ? cluster_rank() : 0;
    const int unit = (int)(gridDim.x / kCtas) - 1 - (int)(blockIdx.x / kCtas);  // tile or pair
    const int qt = unit * kCtas + (int)rank, kvh = blockIdx.y, sp = blockIdx.z;
    const int t0 = qt * p.qtile;
    // live queries of this tile; 0 for the second CTA of the last pair when the tile count is odd
    const int nq = max(0, min(p.qtile, p.tokens - t0));
    const int rows_live = nq * p.group;

    const unsigned bar_full = smem_u32(bars), bar_empty = smem_u32(bars + 3);
    const unsigned bar_s = smem_u32(bars + 6), bar_p = smem_u32(bars + 8), bar_o = smem_u32(bars + 10);
    const unsigned bar_x = smem_u32(bars + 12);
    // Barriers of the leader CTA that this CTA signals (its own when there is no pair).
    const unsigned lead_full = kCtas == 2 ? map_to_cta(bar_full, 0) : bar_full;
    const unsigned lead_p = kCtas == 2 ? map_to_cta(bar_p, 0) : bar_p;
    const unsigned peer_abort =
        kCtas == 2 ? map_to_cta(smem_u32(const_cast<int *>(abort_flag)), rank ^ 1) : 0;

    // Key tiles the CTA (pair) walks: its rows see cache rows < pos0 + (last live query + 1).
    const int t_end = min(p.tokens, (unit + 1) * kCtas * p.qtile);
    const int n_tiles_all = (p.pos0 + t_end + kKeyTile - 1) / kKeyTile;
    const int nsp = p.splits < 2 ? 1 : p.splits;
    const int kt_lo = (int)((long long)n_tiles_all * sp / nsp);
    const int kt_hi = (int)((long long)n_tiles_all * (sp + 1) / nsp);
    const int n_tiles = kt_hi - kt_lo;

    if (tid == 0) {
        for (int i = 0; i < kStages; i++) {
            mbar_init(bar_full + 8 * i, 1);
            mbar_init(bar_empty + 8 * i, 1);
        }
        mbar_init(bar_s, 1);
        mbar_init(bar_s + 8, 1);
        // P ready: one arrival per softmax warp of every CTA of the pair (on the leader)
        mbar_init(bar_p, 8 * kCtas);
        mbar_init(bar_p + 8, 8 * kCtas);
        mbar_init(bar_x, 256);
        mbar_init(bar_x + 8, 256);
        mbar_init(bar_o, 1);
        mbar_init(bar_o + 8, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        __syncwarp();
        tmem_alloc<kCtas>(smem_u32(tmem_slot), 512);  // in the pair form: warp 0 of both CTAs
    }

    // The query rows may come from a grid that is still running (a dependent launch can start
    // while the grid before its predecessor has not finished): nothing is read before this.
    griddep_wait();
    // Q tile: f32 -> scaled hi/lo f16 in the swizzled K-major image. Row r = query r/group,
    // head r%group; rows past the live queries are zero. An item is 8 dims of a row; a thread's
    // items are taken in batches whose loads are all issued before the first is converted (one
    // item at a time the loop cost a memory round trip per item: 9.8 us per CTA, measured).
    {
        constexpr int kItems = 128 * (kD / 8);
        constexpr int kPer = (kItems + kTcThreads - 1) / kTcThreads;
        constexpr int kBatch = kPer;   // all of a thread's items: one round trip
#pragma unroll 1
        for (int b0 = 0; b0 < kPer; b0 += kBatch) {
            float4 lo4[kBatch], hi4[kBatch];
#pragma unroll
            for (int j = 0; j < kBatch; j++) {
                const int i = tid + (b0 + j) * kTcThreads;
                const int r = i >> 5, seg = i & 31;
                lo4[j] = hi4[j] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                if (b0 + j < kPer && i < kItems && r < rows_live) {
                    const int qi = r / p.group, hh = r - qi * p.group;
                    const float4 *src = reinterpret_cast<const float4 *>(
                        p.q + ((size_t)(t0 + qi) * p.n_heads + kvh * p.group + hh) * kD + seg * 8);
                    lo4[j] = __ldg(src);
                    hi4[j] = __ldg(src + 1);
                }
            }
#pragma unroll
            for (int j = 0; j < kBatch; j++) {
                const int i = tid + (b0 + j) * kTcThreads;
                if (b0 + j >= kPer || i >= kItems) continue;
                const int r = i >> 5, seg = i & 31;
                const float x[8] = {lo4[j].x, lo4[j].y, lo4[j].z, lo4[j].w,
                                    hi4[j].x, hi4[j].y, hi4[j].z, hi4[j].w};
                unsigned h[4], l[4];
#pragma unroll
                for (int e = 0; e < 4; e++)
                    split_half2(x[2 * e] * p.scale_log2, x[2 * e + 1] * p.scale_log2, h[e], l[e]);
                const int chunk = seg >> 3, col = (seg & 7) * 8;
                const int off = sw128_offset(r, col);
                *reinterpret_cast<uint4 *>(q_smem + chunk * kTileBytes + off) = make_uint4(h[0], h[1], h[2], h[3]);
                *reinterpret_cast<uint4 *>(q_smem + (4 + chunk) * kTileBytes + off) =
                    make_uint4(l[0], l[1], l[2], l[3]);
            }
        }
    }
    // Make the generic-proxy writes of Q visible to the tensor-core (async) proxy.
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    tc_fence_before();
    // Barriers initialised, Q written, TMEM allocated: in every CTA of the pair before any
    // of them signals the other or the leader's MMAs read the peer's shared memory.
    if constexpr (kCtas == 2) cluster_sync_all(); else __syncthreads();
    tc_fence_after();
    const unsigned tmem = *tmem_slot;
    const unsigned tmem_o = tmem;                 // columns [0,256)
    const unsigned tmem_s[2] = {tmem + 256, tmem + 384};
    const int terms = p.single_pass ? 1 : 3;
    constexpr unsigned kIdescS = idesc_f16(128 * kCtas, 128);         // S = Q K^T
    constexpr unsigned kIdescO = idesc_f16(128 * kCtas, 128 * kCtas); // O += P V (per MMA)
    constexpr int kHalf = kStageBytes / 2;   // low plane of a ring slot

    if (warp == 8) {
        // ---------------------------------------------------------------- TMA producer
        if (lane == 0 && n_tiles > 0) {
            unsigned n = 0;  // chunks issued
            bool ok = true;
            // (the staged image, the scratch and the output rows belong to the previous grids:
            // every thread waited for them before the query tile was read)
            // Takes the next ring slot once the MMAs that read it have completed and arms its
            // full barrier; in a pair only the leader arms, with both CTAs' bytes (the peer's
            // copies complete on the leader's barrier).
            auto acquire = [&](unsigned &dst, unsigned &full) {
                const unsigned stage = n % kStages, phase = (n / kStages) & 1;
                ok = ok && mbar_wait(bar_empty + 8 * stage, phase ^ 1, abort_flag, peer_abort, p.status, 1);
                if (!ok) return;
                dst = smem_u32(ring + stage * kStageBytes);
                full = lead_full + 8 * stage;
                if (rank == 0)
                    mbar_arrive_expect_tx(bar_full + 8 * stage,
                                          kCtas * (p.single_pass ? kStageBytes / 2 : kStageBytes));
                n++;
            };
            auto load_k = [&](int kt) {
                unsigned dst = 0, full = 0;
                if constexpr (kCtas == 1) {
                    // slot = 128 keys x 64 dims (hi, lo)
                    for (int c = 0; c < 4 && ok; c++) {
                        acquire(dst, full);
                        if (!ok) return;
                        const int y = kvh * p.lpad + kt * kKeyTile;
                        tma_load_2d<1>(dst, &map_k_hi, c * 64, y, full);
                        if (!p.single_pass) tma_load_2d<1>(dst + kHalf, &map_k_lo, c * 64, y, full);
                    }
                } else {
                    // slot = this CTA's 64 keys x two 64-dim chunks (hi c, hi c+1, lo c, lo c+1)
                    for (int cp = 0; cp < 2 && ok; cp++) {
                        acquire(dst, full);
                        if (!ok) return;
                        const int y = kvh * p.lpad + kt * kKeyTile + 64 * (int)rank;
                        for (int cc = 0; cc < 2; cc++) {
                            const int x = (2 * cp + cc) * 64;
                            tma_load_2d<2>(dst + cc * (kHalf / 2), &map_k_hi, x, y, full);
                            if (!p.single_pass)
                                tma_load_2d<2>(dst + kHalf + cc * (kHalf / 2), &map_k_lo, x, y, full);
                        }
                    }
                }
            };
            auto load_v = [&](int kt) {
                unsigned dst = 0, full = 0;
                // slot = 128 dims x 64 keys (hi, lo); a pair CTA loads only its half of the dims
                for (int kc = 0; kc < 2 && ok; kc++)
                    for (int dh = 0; dh < (kCtas == 1 ? 2 : 1) && ok; dh++) {
                        acquire(dst, full);
                        if (!ok) return;
                        const int x = kt * kKeyTile + kc * 64;
                        const int y = kvh * kD + (kCtas == 1 ? dh : (int)rank) * 128;
                        tma_load_2d<kCtas>(dst, &map_vt_hi, x, y, full);
                        if (!p.single_pass) tma_load_2d<kCtas>(dst + kHalf, &map_vt_lo, x, y, full);
                    }
            };
            load_k(kt_lo);
            for (int kt = kt_lo; kt < kt_hi && ok; kt++) {
                if (kt + 1 < kt_hi) load_k(kt + 1);
                load_v(kt);
            }
            if (!ok && rank == 0) {
                // Let copies already in flight land before the CTA's shared memory is released
                // (the leader's barriers count the peer's copies too, and the peer stays
                // resident until the leader reaches the closing cluster barrier).
                for (unsigned i = (n > kStages ? n - kStages : 0); i < n; i++)
                    for (unsigned spin = 0; spin < kSpinLimit; spin++)
                        if (mbar_try_wait(bar_full + 8 * (i % kStages), (i / kStages) & 1)) break;
            }
        }
    } else if (warp == 9) {
        // ---------------------------------------------------------------- MMA issuer
        if (lane == 0 && n_tiles > 0 && rank == 0) {
            unsigned n = 0;  // ring slots consumed
            bool ok = true;
            const unsigned q_addr = smem_u32(q_smem);
            // Waits for ring slot n to be full (in a pair: both CTAs' halves) and returns its base.
            auto slot = [&](int code) -> unsigned {
                const unsigned stage = n % kStages, phase = (n / kStages) & 1;
                ok = mbar_wait(bar_full + 8 * stage, phase, abort_flag, peer_abort, p.status, code);
                if (ok) tc_fence_after();
                return smem_u32(ring + stage * kStageBytes);
            };
            auto release = [&]() {  // the slot is free once the MMAs issued so far are done
                tc_commit<kCtas>(bar_empty + 8 * (n % kStages));
                n++;
            };
            // The issuing thread is a serial instruction stream: an MMA of N = 128 keeps the
            // tensor pipe busy for only ~64 cycles, so every instruction between two MMAs
            // counts. Descriptors are therefore formed once per 64-element chunk and advanced
            // by adding the 16-byte-unit offset of the k step to their low word.
            // S += Q[:, 64-dim chunk c] K[:, chunk c]^T with the K chunk (hi at b_hi, lo at b_lo)
            auto qk_chunk = [&](unsigned d, int c, unsigned b_hi, unsigned b_lo) {
                const unsigned a_hi = q_addr + c * kTileBytes, a_lo = a_hi + 4 * kTileBytes;
                const unsigned da[2] = {desc_lo_sw128(a_hi), desc_lo_sw128(a_lo)};
                const unsigned db[2] = {desc_lo_sw128(b_hi), desc_lo_sw128(b_lo)};
#pragma unroll
                for (int term = 0; term < 3; term++) {
                    if (term < terms) {
                        const unsigned a = da[term == 1], b = db[term == 2];
#pragma unroll
                        for (int k16 = 0; k16 < 4; k16++)
                            tc_mma_ss<kCtas>(d, desc_from(a + 2 * k16), desc_from(b + 2 * k16), kIdescS,
                                             (c | term | k16) != 0);
                    }
                }
            };
            auto qk = [&](int i) {  // i = tile index relative to kt_lo
                const unsigned d = tmem_s[i & 1];
                // (unrolled: the chunk index decides at compile time which MMA overwrites S)
                if constexpr (kCtas == 1) {
#pragma unroll
                    for (int c = 0; c < 4; c++) {
                        if (!ok) break;
                        const unsigned b = slot(2);
                        if (!ok) break;
                        qk_chunk(d, c, b, b + kHalf);
                        release();
                    }
                } else {
#pragma unroll
                    for (int cp = 0; cp < 2; cp++) {
                        if (!ok) break;
                        const unsigned b = slot(2);
                        if (!ok) break;
#pragma unroll
                        for (int cc = 0; cc < 2; cc++)
                            qk_chunk(d, 2 * cp + cc, b + cc * (kHalf / 2), b + kHalf + cc * (kHalf / 2));
                        release();
                    }
                }
                if (ok) tc_commit<kCtas>(bar_s + 8 * (i & 1));
            };
            auto pv = [&](int i) {
                const unsigned a_base = tmem_s[i & 1];
                // the first MMA of the first tile, and of every tile that follows a flush of O to
                // memory, overwrites the accumulator
                const unsigned later = (i % kFlushTiles) != 0;
#pragma unroll
                for (int kc = 0; kc < 2; kc++)
#pragma unroll
                    for (int dh = 0; dh < (kCtas == 1 ? 2 : 1); dh++) {
                        if (!ok) break;
                        const unsigned b_hi = slot(3), b_lo = b_hi + kHalf;
                        if (!ok) break;
                        // single CTA: 128 output dims per slot; pair: all 256 (half from each CTA)
                        const unsigned d = tmem_o + dh * 128;
                        const unsigned db[2] = {desc_lo_sw128(b_hi), desc_lo_sw128(b_lo)};
                        const unsigned a0 = a_base + kc * 64;
#pragma unroll
                        for (int term = 0; term < 3; term++) {
                            if (term < terms) {
                                const unsigned b = db[term == 2];
#pragma unroll
                                for (int k16 = 0; k16 < 4; k16++) {
                                    // P of keys [16*(4kc+k16), +16): hi pairs in 8 columns, lo in the next 8
                                    const unsigned a = a0 + k16 * 16 + (term == 1 ? 8 : 0);
                                    tc_mma_ts<kCtas>(d, a, desc_from(b + 2 * k16), kIdescO,
                                                     (kc | term | k16) != 0 ? 1u : later);
                                }
                            }
                        }
                        release();
                    }
                if (ok) tc_commit<kCtas>(bar_o + 8 * (i & 1));
            };
            qk(0);
            for (int i = 0; i < n_tiles && ok; i++) {
                if (i + 1 < n_tiles) qk(i + 1);
                if (!ok) break;
                ok = mbar_wait(bar_p + 8 * (i & 1), (i >> 1) & 1, abort_flag, peer_abort, p.status, 4);
                if (!ok) break;
                tc_fence_after();
                pv(i);
            }
        }
    } else {
        // ---------------------------------------------------------------- softmax + epilogue
        // Two threads per row: thread (row, half) owns score columns [64*half, +64) of the
        // tile and output columns [128*half, +128). The halves of a row meet once per tile
        // through shared memory and an mbarrier (bounded wait) to agree on the row maximum.
        const int r = tid & 127, half = tid >> 7;           // row = TMEM lane
        const unsigned lane_addr = (unsigned)((warp & 3) * 32) << 16;
        const int qi = min(r / p.group, nq - 1);            // dead rows shadow a live query
        const int kmax = p.pos0 + t0 + qi;                  // last visible cache row
        float m_used = -INFINITY, l = 0.0f;
        float m_glob = -INFINITY;   // reference maximum of the part of O already moved to memory
        bool ok = true;
        unsigned v[32];
        // where this thread's half row of the output (or of the slice's partial) lives
        const bool live = r < rows_live;
        const int rq = r / p.group, rh = r - rq * p.group;
        const int h = kvh * p.group + rh;
        const bool norm = p.splits < 2;
        const size_t slot = ((size_t)sp * p.qslots + (t0 + rq)) * p.n_heads + h;
        float *const dst = (norm ? p.out + ((size_t)(t0 + rq) * p.n_heads + h) * kD : p.part_acc + slot * kD) +
                           128 * half;
        // x-th meeting of the two halves: returns the other half's value
        auto meet = [&](int x, float mine, float &other) -> bool {
            float *buf = xch + (x & 1) * 256;
            buf[half * 128 + r] = mine;
            mbar_arrive(bar_x + 8 * (x & 1));
            if (!mbar_wait(bar_x + 8 * (x & 1), (x >> 1) & 1, abort_flag, peer_abort, p.status, 8)) return false;
            other = buf[(half ^ 1) * 128 + r];
            return true;
        };
        for (int i = 0; i < n_tiles && ok; i++) {
            const int key0 = (kt_lo + i) * kKeyTile + 64 * half;
            const unsigned s_addr = tmem_s[i & 1] + lane_addr + 64 * half;
            // (votes keep the warp together: the TMEM accesses below are warp-collective)
            ok = __all_sync(0xffffffffu, mbar_wait(bar_s + 8 * (i & 1), (i >> 1) & 1, abort_flag,
                                                   peer_abort, p.status, 5));
            if (!ok) break;
            tc_fence_after();
            // pass 1: maximum over this thread's visible keys, then over the row
            float m_half = -INFINITY;
#pragma unroll
            for (int j = 0; j < 2; j++) {
                tmem_ld32(s_addr + 32 * j, v);
#pragma unroll
                for (int e = 0; e < 32; e++)
                    if (key0 + 32 * j + e <= kmax) m_half = fmaxf(m_half, __uint_as_float(v[e]));
            }
            float m_other;
            ok = __all_sync(0xffffffffu, meet(i, m_half, m_other));
            if (!ok) break;
            const float m_new = fmaxf(m_used, fmaxf(m_half, m_other));
            // Rescale O only when the maximum moved by more than the threshold (P <= 2^8
            // otherwise); the decision is per warp because the TMEM accesses are collective
            // (both halves of a row see the same maxima, so they decide alike).
            const bool flush = i > 0 && (i % kFlushTiles) == 0;   // the same in every thread of the pair
            const bool want = !flush && (i > 0) && (m_new > m_used + kRescaleThreshold ||
                                                    (m_used == -INFINITY && m_new > -INFINITY));
            if (i == 0) m_used = m_new;
            if (flush) {
                // O (relative to m_used) leaves TMEM: memory += O, in f32, and PV(i) starts afresh
                ok = mbar_wait(bar_o + 8 * ((i - 1) & 1), ((i - 1) >> 1) & 1, abort_flag, peer_abort, p.status, 6);
                if (!__all_sync(0xffffffffu, ok)) { ok = false; break; }
                tc_fence_after();
                const bool first = m_glob == -INFINITY;
                const float cg = first ? 0.0f : exp2f(m_glob - m_used);
#pragma unroll 1
                for (int j = 0; j < 4; j++) {
                    tmem_ld32(tmem_o + lane_addr + 128 * half + 32 * j, v);
                    if (live) {
#pragma unroll
                        for (int e = 0; e < 32; e += 4) {
                            float4 *at = reinterpret_cast<float4 *>(dst + 32 * j + e);
                            float4 w = make_float4(__uint_as_float(v[e]), __uint_as_float(v[e + 1]),
                                                   __uint_as_float(v[e + 2]), __uint_as_float(v[e + 3]));
                            if (!first) {
                                const float4 g = *at;
                                w.x = fmaf(g.x, cg, w.x);
                                w.y = fmaf(g.y, cg, w.y);
                                w.z = fmaf(g.z, cg, w.z);
                                w.w = fmaf(g.w, cg, w.w);
                            }
                            *at = w;
                        }
                    }
                }
                tc_fence_before();
                m_glob = m_used;
                l *= (m_used == -INFINITY) ? 0.0f : exp2f(m_used - m_new);
                m_used = m_new;
            }
            if (__any_sync(0xffffffffu, want)) {
                ok = mbar_wait(bar_o + 8 * ((i - 1) & 1), ((i - 1) >> 1) & 1, abort_flag, peer_abort, p.status, 6);
                if (!__all_sync(0xffffffffu, ok)) { ok = false; break; }
                tc_fence_after();
                const float corr = (m_used == -INFINITY) ? 0.0f : exp2f(m_used - m_new);
#pragma unroll 1
                for (int j = 0; j < 4; j++) {
                    tmem_ld32(tmem_o + lane_addr + 128 * half + 32 * j, v);
#pragma unroll
                    for (int e = 0; e < 32; e++) v[e] = __float_as_uint(__uint_as_float(v[e]) * corr);
                    tmem_st32(tmem_o + lane_addr + 128 * half + 32 * j, v);
                }
                tmem_wait_st();
                l *= corr;
                m_used = m_new;
            }
            // pass 2: P = exp2(S - m), written over S as f16 hi/lo pairs per 16-key step
#pragma unroll 1
            for (int j = 0; j < 2; j++) {
                tmem_ld32(s_addr + 32 * j, v);
                unsigned o[32];
#pragma unroll
                for (int hh = 0; hh < 2; hh++) {
#pragma unroll
                    for (int e = 0; e < 8; e++) {
                        const int ka = hh * 16 + 2 * e;
                        const bool va = key0 + 32 * j + ka <= kmax, vb = key0 + 32 * j + ka + 1 <= kmax;
                        const float pa = va ? exp2f(__uint_as_float(v[ka]) - m_used) : 0.0f;
                        const float pb = vb ? exp2f(__uint_as_float(v[ka + 1]) - m_used) : 0.0f;
                        l += pa + pb;
                        split_half2(pa, pb, o[hh * 16 + e], o[hh * 16 + 8 + e]);
                    }
                }
                tmem_st32(s_addr + 32 * j, o);
            }
            tmem_wait_st();
            tc_fence_before();
            // one arrival per warp, on the CTA that issues the MMAs
            __syncwarp();
            if (lane == 0) {
                if constexpr (kCtas == 2) mbar_arrive_cluster(lead_p + 8 * (i & 1));
                else mbar_arrive(bar_p + 8 * (i & 1));
            }
        }
        // epilogue: the row sum is the two halves' sums; O / l (or the raw partial)
        float l_other = 0.0f;
        if (ok) ok = meet(n_tiles, l, l_other);
        l += l_other;
        if (ok && n_tiles > 0) {
            ok = mbar_wait(bar_o + 8 * ((n_tiles - 1) & 1), ((n_tiles - 1) >> 1) & 1, abort_flag,
                           peer_abort, p.status, 7);
        }
        ok = __all_sync(0xffffffffu, ok);
        // O leaves TMEM through shared memory: a thread owns half a row (lane = row), so its own
        // stores to memory would be 16-byte pieces 1 KB apart (8,192 write transactions per CTA,
        // 6.3 us measured); staged, whole 1 KB rows leave by bulk copies, which a CTA only has
        // to see read, not written, before it makes room for the next one (rows that add to a
        // part already in memory, or take the output gate, are written by the warps instead).
        // The query tile and the ring are dead by now (every MMA of the pair has completed, every
        // copy was consumed).
        const bool bulk_rows = n_tiles <= kFlushTiles && !(norm && p.gate);   // the same in every thread
        constexpr int kPitch = kD + 4;                       // floats; 16-byte stores of 8 rows hit 8 bank groups
        float *const stage = reinterpret_cast<float *>(smem);
        float *const row_scale = stage + 128 * kPitch;        // per row: {weight of the flushed part (< 0: none), 1 / l}
        if (ok) {
            griddep_wait();   // (already satisfied unless the CTA had no key tiles to wait for)
            tc_fence_after();
            const float inv = norm ? (l > 0.0f ? 1.0f / l : 0.0f) : 1.0f;
#pragma unroll 1
            for (int j = 0; j < 4; j++) {
                if (n_tiles > 0) {
                    tmem_ld32(tmem_o + lane_addr + 128 * half + 32 * j, v);
                } else {
#pragma unroll
                    for (int e = 0; e < 32; e++) v[e] = 0u;
                }
                if (live) {
                    float *at = stage + r * kPitch + 128 * half + 32 * j;
                    const float pre = bulk_rows ? inv : 1.0f;
#pragma unroll
                    for (int e = 0; e < 32; e += 4)
                        *reinterpret_cast<float4 *>(at + e) =
                            make_float4(__uint_as_float(v[e]) * pre, __uint_as_float(v[e + 1]) * pre,
                                        __uint_as_float(v[e + 2]) * pre, __uint_as_float(v[e + 3]) * pre);
                }
            }
            if (bulk_rows) fence_async_shared();   // these rows are read by the bulk copies below
            if (live && half == 0) {
                const bool flushed = m_glob != -INFINITY;   // part of O is in memory already
                row_scale[2 * r] = flushed ? exp2f(m_glob - m_used) : -1.0f;
                row_scale[2 * r + 1] = inv;
                if (!norm) {
                    p.part_ml[slot * 2] = m_used;
                    p.part_ml[slot * 2 + 1] = l;
                }
            }
        }
        // (the eight softmax warps; a warp that gave up still arrives, and nothing is written then)
        asm volatile("bar.sync 1, 256;" ::: "memory");
        if (*abort_flag == 0 && bulk_rows) {
            if (lane == 0) {
                for (int rr = warp; rr < rows_live; rr += 8) {
                    const int q2 = rr / p.group, h2 = kvh * p.group + (rr - q2 * p.group);
                    const size_t row = norm ? ((size_t)(t0 + q2) * p.n_heads + h2)
                                            : (((size_t)sp * p.qslots + (t0 + q2)) * p.n_heads + h2);
                    bulk_store((norm ? p.out : p.part_acc) + row * kD, smem_u32(stage + rr * kPitch), kD * 4);
                }
                bulk_store_commit_wait_read();
            }
        } else if (*abort_flag == 0) {
            for (int rr = warp; rr < rows_live; rr += 8) {
                const int q2 = rr / p.group, h2 = kvh * p.group + (rr - q2 * p.group);
                const size_t row = norm ? ((size_t)(t0 + q2) * p.n_heads + h2)
                                        : (((size_t)sp * p.qslots + (t0 + q2)) * p.n_heads + h2);
                float *const drow = (norm ? p.out : p.part_acc) + row * kD;
                const float *const grow = (norm && p.gate) ? p.gate + row * kD : nullptr;
                const float cg = row_scale[2 * rr], inv = row_scale[2 * rr + 1];
#pragma unroll
                for (int c = 0; c < 2; c++) {
                    const int col = 128 * c + 4 * lane;
                    float4 w = *reinterpret_cast<const float4 *>(stage + rr * kPitch + col);
                    if (cg >= 0.0f) {
                        const float4 g = *reinterpret_cast<const float4 *>(drow + col);
                        w.x = fmaf(g.x, cg, w.x);
                        w.y = fmaf(g.y, cg, w.y);
                        w.z = fmaf(g.z, cg, w.z);
                        w.w = fmaf(g.w, cg, w.w);
                    }
                    w.x *= inv;
                    w.y *= inv;
                    w.z *= inv;
                    w.w *= inv;
                    if (grow) {   // the layer's output gate, applied where the row is produced
                        const float4 g = *reinterpret_cast<const float4 *>(grow + col);
                        w.x *= 1.0f / (1.0f + expf(-g.x));
                        w.y *= 1.0f / (1.0f + expf(-g.y));
                        w.z *= 1.0f / (1.0f + expf(-g.z));
                        w.w *= 1.0f / (1.0f + expf(-g.w));
                    }
                    *reinterpret_cast<float4 *>(drow + col) = w;
                }
            }
        }
    }

    // Nothing of the pair may still be in flight towards either CTA (MMAs reading the peer's
    // shared memory, barrier arrivals, copies) when one of them releases its TMEM and exits.
    tc_fence_before();
    if constexpr (kCtas == 2) cluster_sync_all(); else __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        tmem_dealloc<kCtas>(tmem, 512);
    }
}

// 2D f16 tensor [rows][cols] (cols contiguous), box `box_rows` rows x 64 cols, 128-byte swizzle.
int make_map(CUtensorMap *map, void *base, uint64_t cols, uint64_t rows, uint32_t box_rows) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return fail(HIPML_ERR_INVALID_ARGUMENT, "cuTensorMapEncodeTiled is not available");
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {cols * 2};
    const cuuint32_t box[2] = {64, box_rows};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, base, dims, strides, box, elem,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(HIPML_ERR_INVALID_ARGUMENT, "cuTensorMapEncodeTiled failed: %d", (int)r);
    return 0;
}

}  // namespace

size_t chunk_tc_workspace_bytes(int n_kv, int n_keys) {
    const size_t lpad = ((size_t)n_keys + kKeyTile - 1) / kKeyTile * kKeyTile;
    return 4 * (size_t)n_kv * lpad * kD * sizeof(__half);
}

// Stages cache rows [key_from, key_to) into a workspace laid out for `cap` keys per head
// (cap a multiple of 128, >= key_to): whole 64-key tiles are rewritten, and rows from key_to
// up to the next multiple of 128 are zero-filled so the last key tile is finite.
int launch_chunk_stage(cudaStream_t stream, const void *k_cache, const void *v_cache, int n_kv,
                       int kv_dtype, int stride, int key_from, int key_to, int cap,
                       void *workspace) {
    const size_t plane = (size_t)n_kv * cap * kD;
    __half *ws = reinterpret_cast<__half *>(workspace);
    StageParams sp;
    sp.k = k_cache;
    sp.v = v_cache;
    sp.k_hi = ws;
    sp.k_lo = ws + plane;
    sp.vt_hi = ws + 2 * plane;
    sp.vt_lo = ws + 3 * plane;
    sp.n_kv = n_kv;
    sp.n_keys = key_to;
    sp.lpad = cap;
    sp.kv_dtype = kv_dtype;
    sp.stride = stride;
    sp.tile0 = key_from / 64;
    const int tile_end = (key_to + kKeyTile - 1) / kKeyTile * kKeyTile / 64;
    if (tile_end <= sp.tile0) return 0;
    return launch_pdl(attn_chunk_stage, dim3(tile_end - sp.tile0, n_kv, 3), dim3(256), 0, stream, 1, sp);
}

// Launches the tensor-core kernel over a workspace staged for `cap` keys per head.
// variant bit 0: single-pass precision (hi*hi only); bit 1: the single-CTA form instead of
// CTA pairs. Shapes are validated by the caller.
int launch_chunk_tc(cudaStream_t stream, const float *q, float *out, float *part_acc,
                    float *part_ml, int n_heads, int n_kv, int pos0, int tokens, int cap,
                    int splits, int variant, void *workspace, int *status, const float *gate) {
    const size_t plane = (size_t)n_kv * cap * kD;
    __half *ws = reinterpret_cast<__half *>(workspace);
    const bool pair = (variant & 2) == 0;
    const int single_pass = variant & 1;
    int rc;
    CUtensorMap mk_hi, mk_lo, mv_hi, mv_lo;
    const uint32_t k_box = pair ? 64 : 128;   // a pair CTA loads its 64 keys of a 128-key tile
    if ((rc = make_map(&mk_hi, ws, kD, (uint64_t)n_kv * cap, k_box))) return rc;
    if ((rc = make_map(&mk_lo, ws + plane, kD, (uint64_t)n_kv * cap, k_box))) return rc;
    if ((rc = make_map(&mv_hi, ws + 2 * plane, cap, (uint64_t)n_kv * kD, 128))) return rc;
    if ((rc = make_map(&mv_lo, ws + 3 * plane, cap, (uint64_t)n_kv * kD, 128))) return rc;

    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(attn_chunk_tc<1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             kSmemBytes);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(attn_chunk_tc<2>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     kSmemBytes);
        if (e != cudaSuccess) return (int)e;
        configured[dev] = true;
    }

    ChunkTcParams p;
    p.q = q;
    p.out = out;
    p.part_acc = part_acc;
    p.part_ml = part_ml;
    p.status = status;
    p.n_heads = n_heads;
    p.n_kv = n_kv;
    p.group = n_heads / n_kv;
    p.pos0 = pos0;
    p.tokens = tokens;
    p.lpad = cap;
    p.qtile = 128 / p.group;
    p.scale_log2 = (1.0f / sqrtf((float)kD)) * 1.4426950408889634f;
    p.splits = splits;
    p.qslots = (tokens + 31) / 32 * 32;
    p.single_pass = single_pass;
    p.gate = gate;
    const int nsp = splits < 2 ? 1 : splits;
    const int qtiles = (tokens + p.qtile - 1) / p.qtile;
    if (!pair) {
        return launch_pdl(attn_chunk_tc<1>, dim3(qtiles, n_kv, nsp), dim3(kTcThreads), (size_t)kSmemBytes,
                          stream, 1, mk_hi, mk_lo, mv_hi, mv_lo, p);
    }
    // Clusters of two CTAs along x: consecutive query tiles of one KV head (an odd tile
    // count leaves the last pair's second CTA without live queries).
    return launch_pdl(attn_chunk_tc<2>, dim3((qtiles + 1) / 2 * 2, n_kv, nsp), dim3(kTcThreads),
                      (size_t)kSmemBytes, stream, 2, mk_hi, mk_lo, mv_hi, mv_lo, p);
}

}  // namespace hipml
