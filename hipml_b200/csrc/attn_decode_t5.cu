// Split-K flash-decode over the q8_0 cache on tcgen05 (head_dim 256): the conversion of the
// cache bytes is decoupled from the contractions.
//
// A persistent CTA (one per SM) walks (KV head, split[, slot]) tasks in 128-key tiles.
//   * Group A (warps 0-3, thread = key of the tile) loads its key's K row (272 B) straight
//     into registers, converts the int8 codes to f16 (exact) and stores them as the K-major,
//     128B-swizzled A operand; the MMA thread issues S^T[key][head] = K Q^T per 32-dim block
//     (tcgen05.mma kind::f16, M = 128 keys, N = 16 = 6 heads x (hi, lo) + padding, one
//     accumulator per block); group A reads the eight block partials of its key from TMEM,
//     applies the K scales in f32, runs the online softmax across the tile and writes the
//     weights as f16 hi/lo rows of the P operand.
//   * Group B (warps 4-7, thread = key) does the same for V, folding the block scale into the
//     value as an exact f16 hi + lo pair (a dequantised value has at most 18 significant
//     bits), stored [key][dim], which the MMA reads as an M-major A operand:
//     O^T[dim][head] += V^T P^T (M = 2 x 128 dims, N = 16, K = 128 keys).
//   * Warp 8 issues the MMAs. TMEM: O^T 2 x 16 columns, S^T 8 x 16 columns.
// The next tile's rows are requested (17 x 16-byte loads per thread) before the current tile's
// scores are awaited, across task boundaries too, so HBM latency is covered by the softmax.
// Every mbarrier wait is bounded and reports through the device status word.
//
// CPU definition: crates/hipml-core/src/ops.rs:449-518. Kernel replaced:
// crates/hipml-kernels/kernels/attn_decode_kv_w.hip:92-285 (selector 5 of
// hipml_attn_decode_kv; partial layout as for the other bodies).
#include "params.cuh"
#include "tc_ptx.cuh"

namespace hipml {

namespace {

using namespace ptx;

constexpr int kT = 128;                  // keys per tile
constexpr int kRowB = 272;               // q8 row bytes at head_dim 256
constexpr int kChunk = 16384;            // [128 rows][64 f16] swizzled tile
constexpr int kOffK = 0;                 // K f16: 4 chunks (64 dims each)
constexpr int kOffVh = 4 * kChunk;       // V hi
constexpr int kOffVl = 8 * kChunk;       // V lo
constexpr int kOffQt = 12 * kChunk;      // Q^T: 4 chunks of [16 rows][64 dims] (2 KB each)
constexpr int kOffPt = kOffQt + 4 * 2048;  // P^T: 2 chunks of [16 rows][64 keys]
constexpr int kOffRed = kOffPt + 2 * 2048; // reduction scratch: max [2][4][8] + sum [2][4][8] floats
constexpr int kOffBar = kOffRed + 512;
constexpr int kSmem = kOffBar + 128 + 1024;  // + alignment slack
constexpr int kThreadsT5 = 288;
constexpr float kLazy = 8.0f;

constexpr unsigned kIdescQK = idesc_f16(128, 16, 0, 0);
constexpr unsigned kIdescPV = idesc_f16(128, 16, 1, 0);

struct Tile {
    int task, tile;        // task index (kvh * splits + split, + slot * n_kv * splits), tile in task
    int kvh, split, slot;
    int key0, nvalid;      // first cache row of the tile, live rows in it
    int first, last;       // first / last tile of its task
};

// The (task, tile) sequence of one persistent CTA.
struct Walker {
    const DecodeParams &p;
    int slots, tasks, cur_task, cur_tile, ntiles, lo, hi;
    __device__ Walker(const DecodeParams &p_, int slots_) : p(p_), slots(slots_) {
        tasks = p.n_kv * p.splits * slots;
        cur_task = blockIdx.x - gridDim.x;
        cur_tile = 0;
        ntiles = 0;
        lo = hi = 0;
    }
    __device__ void open_task() {
        const int per_slot = p.n_kv * p.splits;
        const int slot = cur_task / per_slot, rem = cur_task - slot * per_slot;
        const int split = rem % p.splits;
        const int len = p.len[slot * p.len_stride + p.len_offset];
        const int span = p.by_stride ? p.stride : len;
        const int per = (span + p.splits - 1) / p.splits;
        lo = min(split * per, len);
        hi = min(lo + per, len);
        ntiles = max((hi - lo + kT - 1) / kT, 1);  // an empty task still walks one empty tile
        cur_tile = 0;
    }
    // Advances to the next tile; false when the CTA's work is done.
    __device__ bool next(Tile &t) {
        if (cur_task >= 0 && cur_tile + 1 < ntiles) {
            cur_tile++;
        } else {
            cur_task += gridDim.x;
            if (cur_task >= tasks) return false;
            open_task();
        }
        const int per_slot = p.n_kv * p.splits;
        t.task = cur_task;
        t.tile = cur_tile;
        t.slot = cur_task / per_slot;
        const int rem = cur_task - t.slot * per_slot;
        t.kvh = rem / p.splits;
        t.split = rem - t.kvh * p.splits;
        t.key0 = lo + cur_tile * kT;
        t.nvalid = max(min(kT, hi - t.key0), 0);
        t.first = cur_tile == 0;
        t.last = cur_tile == ntiles - 1;
        return true;
    }
};

// This thread's row of the tile as 17 x 16 bytes (zeros past the live rows).
struct Row {
    uint4 v[17];
};

__device__ __forceinline__ void load_row(Row &r, const unsigned char *cache, const DecodeParams &p,
                                         const Tile &t, int key) {
    if (key < t.nvalid) {
        const uint4 *src = reinterpret_cast<const uint4 *>(
            cache + (size_t)t.slot * p.kv_slot_bytes + q8_row_offset(t.kvh, p.stride, t.key0 + key, 256));
#pragma unroll
        for (int i = 0; i < 17; i++) r.v[i] = __ldg(src + i);
    } else {
#pragma unroll
        for (int i = 0; i < 17; i++) r.v[i] = make_uint4(0, 0, 0, 0);
    }
}

__device__ __forceinline__ unsigned row_word(const Row &r, int w) {
    const uint4 &q = r.v[w >> 2];
    return (w & 3) == 0 ? q.x : (w & 3) == 1 ? q.y : (w & 3) == 2 ? q.z : q.w;
}

// f16 bits of the scale of block B (bytes 34B, 34B+1 of the row).
template <int B>
__device__ __forceinline__ unsigned short row_scale_bits(const Row &r) {
    constexpr int byte = 34 * B;
    const unsigned w = row_word(r, byte >> 2);
    return (byte & 3) == 0 ? (unsigned short)(w & 0xffff) : (unsigned short)(w >> 16);
}

// Codes j, j+1 (j even) of block B as an exact half2.
template <int B>
__device__ __forceinline__ __half2 row_codes2(const Row &r, int j) {
    const int byte = 34 * B + 2 + j;  // even; never straddles a word
    const unsigned w = row_word(r, byte >> 2) ^ 0x80808080u;
    const unsigned h = __byte_perm(w, 0x64646464u, (byte & 3) == 0 ? 0x4140 : 0x4342);
    return __hsub2(*reinterpret_cast<const __half2 *>(&h), __half2half2(__ushort_as_half(0x6480)));
}

__device__ __forceinline__ unsigned h2u(__half2 h) { return *reinterpret_cast<unsigned *>(&h); }

// K: codes only (the scale is applied to the block's partial dot product in f32).
template <int B>
__device__ __forceinline__ void convert_k_block(const Row &r, unsigned char *kf16, int key) {
#pragma unroll
    for (int u = 0; u < 4; u++) {
        const uint4 o = make_uint4(h2u(row_codes2<B>(r, 8 * u)), h2u(row_codes2<B>(r, 8 * u + 2)),
                                   h2u(row_codes2<B>(r, 8 * u + 4)), h2u(row_codes2<B>(r, 8 * u + 6)));
        *reinterpret_cast<uint4 *>(kf16 + (B >> 1) * kChunk + sw128_offset(key, (B & 1) * 32 + 8 * u)) = o;
    }
}

// V: scale * code as an exact f16 high + low pair.
template <int B>
__device__ __forceinline__ void convert_v_block(const Row &r, unsigned char *vhi, unsigned char *vlo,
                                                int key) {
    const __half2 d = __half2half2(__ushort_as_half(row_scale_bits<B>(r)));
#pragma unroll
    for (int u = 0; u < 4; u++) {
        __half2 hi[4], lo[4];
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const __half2 c = row_codes2<B>(r, 8 * u + 2 * e);
            hi[e] = __hmul2(d, c);
            lo[e] = __hfma2(d, c, __hneg2(hi[e]));
        }
        const int off = (B >> 1) * kChunk + sw128_offset(key, (B & 1) * 32 + 8 * u);
        *reinterpret_cast<uint4 *>(vhi + off) = make_uint4(h2u(hi[0]), h2u(hi[1]), h2u(hi[2]), h2u(hi[3]));
        *reinterpret_cast<uint4 *>(vlo + off) = make_uint4(h2u(lo[0]), h2u(lo[1]), h2u(lo[2]), h2u(lo[3]));
    }
}

__device__ __forceinline__ void bar_group_a() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// Maximum over the 32 lanes through the integer redux unit (floats mapped to ordered ints).
__device__ __forceinline__ float warp_max_redux(float x) {
    int i = __float_as_int(x);
    i ^= (i >> 31) & 0x7fffffff;
    i = __reduce_max_sync(0xffffffffu, i);
    i ^= (i >> 31) & 0x7fffffff;
    return __int_as_float(i);
}

__global__ void __launch_bounds__(kThreadsT5, 1) attn_decode_kv_t5(DecodeParams p, int slots, int *status) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char *smem =
        reinterpret_cast<unsigned char *>((reinterpret_cast<size_t>(smem_raw) + 1023) & ~(size_t)1023);
    unsigned char *kf16 = smem + kOffK, *vhi = smem + kOffVh, *vlo = smem + kOffVl;
    unsigned char *qt = smem + kOffQt, *pt = smem + kOffPt;
    float *red = reinterpret_cast<float *>(smem + kOffRed);   // [2][4][8]
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + kOffBar);
    // bars: 0 k_full, 1 s_ready, 2 v_full, 3 p_ready, 4..5 o_done[2]
    volatile int *abort_flag = reinterpret_cast<volatile int *>(bars + 8);
    unsigned *tmem_slot = reinterpret_cast<unsigned *>(bars + 9);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const unsigned b_kfull = smem_u32(bars), b_sready = smem_u32(bars + 1), b_vfull = smem_u32(bars + 2);
    const unsigned b_pready = smem_u32(bars + 3), b_odone = smem_u32(bars + 4);
    const int group = p.n_heads / p.n_kv;

    if (tid == 0) {
        mbar_init(b_kfull, 128);
        mbar_init(b_sready, 1);
        mbar_init(b_vfull, 128);
        mbar_init(b_pready, 128);
        mbar_init(b_odone, 1);
        mbar_init(b_odone + 8, 1);
        *abort_flag = 0;
        mbar_init_fence();
    }
    // Q^T and P^T start as zeros: rows 6, 7, 14, 15 (padding) are never written again.
    for (int i = tid; i < (4 * 2048 + 2 * 2048) / 16; i += kThreadsT5)
        reinterpret_cast<uint4 *>(qt)[i] = make_uint4(0, 0, 0, 0);
    if (warp == 0) {
        __syncwarp();
        tmem_alloc(smem_u32(tmem_slot), 256);
    }
    fence_async_shared();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem = *tmem_slot;
    const unsigned tmem_o = tmem, tmem_s = tmem + 32;

    Walker walk(p, slots);
    Tile t;
    unsigned g = 0;  // global tile counter of this CTA

    if (warp < 4) {
        // ------------------------------------------------------------ group A: K, scores, softmax
        const int key = tid;
        const unsigned lane_addr = (unsigned)(warp * 32) << 16;
        Row row;
        bool more = walk.next(t);
        if (more) load_row(row, p.k, p, t, key);
        float m_used[6], l_thr[6];
        bool ok = true;
        while (more && ok) {
            if (t.first) {
#pragma unroll
                for (int h = 0; h < 6; h++) {
                    m_used[h] = -INFINITY;
                    l_thr[h] = 0.0f;
                }
                // Q^T of this task's KV head: rows 0..5 = f16 high part of head h, 8..13 = low part,
                // in log2 units. Two dims per thread.
                const float *q = p.q + (size_t)t.slot * p.q_slot + (size_t)t.kvh * group * 256;
#pragma unroll
                for (int half = 0; half < 2; half++) {
                    const int d = key + 128 * half;
                    for (int h = 0; h < group && h < 6; h++) {
                        const float x = q[h * 256 + d] * p.scale_log2;
                        const __half xh = __float2half_rn(x);
                        const __half xl = __float2half_rn(x - __half2float(xh));
                        unsigned char *base = qt + (d >> 6) * 2048;
                        *reinterpret_cast<__half *>(base + sw128_offset(h, d & 63)) = xh;
                        *reinterpret_cast<__half *>(base + sw128_offset(8 + h, d & 63)) = xl;
                    }
                }
            }
            // K row -> f16 A operand (the previous tile's QK^T has completed: its scores were read)
            convert_k_block<0>(row, kf16, key);
            convert_k_block<1>(row, kf16, key);
            convert_k_block<2>(row, kf16, key);
            convert_k_block<3>(row, kf16, key);
            convert_k_block<4>(row, kf16, key);
            convert_k_block<5>(row, kf16, key);
            convert_k_block<6>(row, kf16, key);
            convert_k_block<7>(row, kf16, key);
            float dk[8];
            dk[0] = half_bits_to_float(row_scale_bits<0>(row));
            dk[1] = half_bits_to_float(row_scale_bits<1>(row));
            dk[2] = half_bits_to_float(row_scale_bits<2>(row));
            dk[3] = half_bits_to_float(row_scale_bits<3>(row));
            dk[4] = half_bits_to_float(row_scale_bits<4>(row));
            dk[5] = half_bits_to_float(row_scale_bits<5>(row));
            dk[6] = half_bits_to_float(row_scale_bits<6>(row));
            dk[7] = half_bits_to_float(row_scale_bits<7>(row));
            fence_async_shared();
            tc_fence_before();  // this thread's reads of the previous scores precede the next QK^T
            mbar_arrive(b_kfull);

            // request the next tile's row now; it lands while the scores are awaited and reduced
            const Tile cur = t;
            more = walk.next(t);
            if (more) load_row(row, p.k, p, t, key);

            ok = mbar_wait(b_sready, g & 1, abort_flag, status, 11);
            if (!ok) break;
            tc_fence_after();
            float s[6] = {0, 0, 0, 0, 0, 0};
#pragma unroll
            for (int j = 0; j < 4; j++) {  // 32 columns = blocks 2j, 2j+1
                unsigned v[32];
                tmem_ld32(tmem_s + lane_addr + 32 * j, v);
#pragma unroll
                for (int h = 0; h < 6; h++) {
                    s[h] += dk[2 * j] * (__uint_as_float(v[h]) + __uint_as_float(v[8 + h]));
                    s[h] += dk[2 * j + 1] * (__uint_as_float(v[16 + h]) + __uint_as_float(v[24 + h]));
                }
            }
            const bool live = key < cur.nvalid;
            // tile maximum per head: redux inside the warp, shared memory across the four warps
            float *rbuf = red + (g & 1) * 32;
#pragma unroll
            for (int h = 0; h < 6; h++) {
                const float mx = warp_max_redux(live ? s[h] : -INFINITY);
                if (lane == 0) rbuf[warp * 8 + h] = mx;
            }
            bar_group_a();
            float m_new[6];
            bool want = false;
#pragma unroll
            for (int h = 0; h < 6; h++) {
                const float mt = fmaxf(fmaxf(rbuf[h], rbuf[8 + h]), fmaxf(rbuf[16 + h], rbuf[24 + h]));
                m_new[h] = fmaxf(m_used[h], mt);
                want = want || m_new[h] > m_used[h] + kLazy || (m_used[h] == -INFINITY && m_new[h] > -INFINITY);
            }
            // the previous tile's PV must be done before P (and O) are touched
            if (g > 0) {
                ok = mbar_wait(b_odone + 8 * ((g - 1) & 1), ((g - 1) >> 1) & 1, abort_flag, status, 12);
                if (!ok) break;
                tc_fence_after();
            }
            if (want) {  // uniform across the CTA: every thread holds the same maxima
                float corr[6];
#pragma unroll
                for (int h = 0; h < 6; h++) {
                    corr[h] = (m_used[h] == -INFINITY) ? 0.0f : exp2f(m_used[h] - m_new[h]);
                    l_thr[h] *= corr[h];
                    m_used[h] = m_new[h];
                }
                if (!cur.first) {
                    unsigned v[32];
                    tmem_ld32(tmem_o + lane_addr, v);
#pragma unroll
                    for (int n = 0; n < 32; n++)
                        if ((n & 7) < 6) v[n] = __float_as_uint(__uint_as_float(v[n]) * corr[n & 7]);
                    tmem_st32(tmem_o + lane_addr, v);
                }
            }
            // weights of this key, f16 high/low rows of P^T
            unsigned char *pbase = pt + (key >> 6) * 2048;
#pragma unroll
            for (int h = 0; h < 6; h++) {
                const float w = live ? exp2f(s[h] - m_used[h]) : 0.0f;
                l_thr[h] += w;
                const __half wh = __float2half_rn(w);
                const __half wl = __float2half_rn(w - __half2float(wh));
                *reinterpret_cast<__half *>(pbase + sw128_offset(h, key & 63)) = wh;
                *reinterpret_cast<__half *>(pbase + sw128_offset(8 + h, key & 63)) = wl;
            }
            fence_async_shared();
            tc_fence_before();
            mbar_arrive(b_pready);

            if (cur.last) {
                // task epilogue: O^T of dims key and 128 + key, then the (max, sum) pair
                ok = mbar_wait(b_odone + 8 * (g & 1), (g >> 1) & 1, abort_flag, status, 13);
                if (!ok) break;
                tc_fence_after();
                unsigned v[32];
                tmem_ld32(tmem_o + lane_addr, v);
                float *rl = red + 64 + ((g & 1) * 32);
#pragma unroll
                for (int h = 0; h < 6; h++) {
                    const float sum = warp_sum(l_thr[h]);
                    if (lane == 0) rl[warp * 8 + h] = sum;
                }
                bar_group_a();
                const size_t per_slot_acc = (size_t)cur.slot * p.acc_slot, per_slot_ml = (size_t)cur.slot * p.ml_slot;
                for (int h = 0; h < group && h < 6; h++) {
                    const int head = cur.kvh * group + h;
                    float *pa = p.part_acc + per_slot_acc + ((size_t)head * p.splits + cur.split) * 256;
                    pa[key] = __uint_as_float(v[h]) + __uint_as_float(v[8 + h]);
                    pa[128 + key] = __uint_as_float(v[16 + h]) + __uint_as_float(v[24 + h]);
                    if (key == h) {
                        float *pm = p.part_ml + per_slot_ml + ((size_t)head * p.splits + cur.split) * 2;
                        pm[0] = m_used[h];
                        pm[1] = rl[h] + rl[8 + h] + rl[16 + h] + rl[24 + h];
                    }
                }
            }
            g++;
        }
    } else if (warp < 8) {
        // ------------------------------------------------------------ group B: V
        const int key = tid - 128;
        Row row;
        bool more = walk.next(t);
        if (more) load_row(row, p.v, p, t, key);
        bool ok = true;
        while (more && ok) {
            if (g > 0) {  // the previous tile's PV has read the V operand
                ok = mbar_wait(b_odone + 8 * ((g - 1) & 1), ((g - 1) >> 1) & 1, abort_flag, status, 14);
                if (!ok) break;
            }
            convert_v_block<0>(row, vhi, vlo, key);
            convert_v_block<1>(row, vhi, vlo, key);
            convert_v_block<2>(row, vhi, vlo, key);
            convert_v_block<3>(row, vhi, vlo, key);
            convert_v_block<4>(row, vhi, vlo, key);
            convert_v_block<5>(row, vhi, vlo, key);
            convert_v_block<6>(row, vhi, vlo, key);
            convert_v_block<7>(row, vhi, vlo, key);
            fence_async_shared();
            mbar_arrive(b_vfull);
            more = walk.next(t);
            if (more) load_row(row, p.v, p, t, key);
            g++;
        }
    } else if (lane == 0) {
        // ------------------------------------------------------------ MMA issuer
        bool ok = true;
        const unsigned a_k = smem_u32(kf16), a_vh = smem_u32(vhi), a_vl = smem_u32(vlo);
        const unsigned b_q = smem_u32(qt), b_p = smem_u32(pt);
        while (ok && walk.next(t)) {
            ok = mbar_wait(b_kfull, g & 1, abort_flag, status, 15);
            if (!ok) break;
            tc_fence_after();
#pragma unroll
            for (int b = 0; b < 8; b++)
#pragma unroll
                for (int kk = 0; kk < 2; kk++) {
                    const unsigned off = ((b & 1) * 2 + kk) * 32;
                    tc_mma_ss(tmem_s + 16 * b, smem_desc(a_k + (b >> 1) * kChunk + off, 16, 1024, 2),
                              smem_desc(b_q + (b >> 1) * 2048 + off, 16, 1024, 2), kIdescQK, kk);
                }
            tc_commit(b_sready);
            ok = mbar_wait(b_vfull, g & 1, abort_flag, status, 16);
            if (!ok) break;
            ok = mbar_wait(b_pready, g & 1, abort_flag, status, 17);
            if (!ok) break;
            tc_fence_after();
#pragma unroll
            for (int mt = 0; mt < 2; mt++)
#pragma unroll
                for (int ks = 0; ks < 8; ks++) {
                    // A = V^T: M-major, 64-dim chunks 16 KB apart, 8-key groups 1 KB apart
                    const unsigned a_off = mt * 2 * kChunk + ks * 2048;
                    const uint64_t bdesc = smem_desc(b_p + (ks >> 2) * 2048 + (ks & 3) * 32, 16, 1024, 2);
                    tc_mma_ss(tmem_o + 16 * mt, smem_desc(a_vh + a_off, kChunk, 1024, 2), bdesc, kIdescPV,
                              !(t.first && ks == 0));
                    tc_mma_ss(tmem_o + 16 * mt, smem_desc(a_vl + a_off, kChunk, 1024, 2), bdesc, kIdescPV, 1);
                }
            tc_commit(b_odone + 8 * (g & 1));
            g++;
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        tmem_dealloc(tmem, 256);
    }
}

}  // namespace

int launch_decode_t5(cudaStream_t stream, const DecodeParams &p, int slots, int *status) {
    static int sms[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) return fail(HIPML_ERR_INVALID_ARGUMENT, "device ordinal %d", dev);
    if (!sms[dev]) {
        cudaError_t e = cudaFuncSetAttribute(attn_decode_kv_t5, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             kSmem);
        if (e != cudaSuccess) return (int)e;
        int n = 0;
        e = cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess) return (int)e;
        sms[dev] = n;
    }
    const int tasks = p.n_kv * p.splits * slots;
    const int grid = tasks < sms[dev] ? tasks : sms[dev];
    attn_decode_kv_t5<<<grid, kThreadsT5, kSmem, stream>>>(p, slots, status);
    return launch_status();
}

}  // namespace hipml
