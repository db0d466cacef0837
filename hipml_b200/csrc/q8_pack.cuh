// q8_0 row assembly shared by the append kernels: quantise eight values per lane into a
// row image in shared memory, and stream a finished image to the cache.
// Format definition: crates/hipml-core/src/kv.rs:187-200.
#pragma once

#include "common.cuh"

namespace hipml {

constexpr int kMaxRowBytes = 8 * kQ8BlockBytes;  // head_dim 256

// Copy a finished row image to global memory with the widest store its
// address and length allow (16 B for head_dim 256, whose rows are 272 B).
__device__ __forceinline__ void row_store(unsigned char *dst, const unsigned char *row,
                                          int row_bytes, int tid, int nthreads) {
    const size_t a = reinterpret_cast<size_t>(dst) | (size_t)row_bytes;
    if ((a & 15) == 0) {
        for (int i = tid; i < row_bytes / 16; i += nthreads)
            reinterpret_cast<uint4 *>(dst)[i] = reinterpret_cast<const uint4 *>(row)[i];
    } else if ((a & 3) == 0) {
        for (int i = tid; i < row_bytes / 4; i += nthreads)
            reinterpret_cast<uint32_t *>(dst)[i] = reinterpret_cast<const uint32_t *>(row)[i];
    } else {
        for (int i = tid; i < row_bytes / 2; i += nthreads)
            reinterpret_cast<unsigned short *>(dst)[i] =
                reinterpret_cast<const unsigned short *>(row)[i];
    }
}

// Eight values of one 32-value block held by one lane (lanes 4b..4b+3 share block b).
__device__ __forceinline__ void q8_put8(const float4 a, const float4 b, int lane,
                                        unsigned char *row) {
    const float x[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    float amax = 0.0f;
#pragma unroll
    for (int j = 0; j < 8; j++) amax = fmaxf(amax, fabsf(x[j]));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    const float d = amax / 127.0f;
    const float id = d > 0.0f ? 1.0f / d : 0.0f;
    unsigned q[8];
#pragma unroll
    for (int j = 0; j < 8; j++) {
        const float r = roundf(x[j] * id);
        q[j] = (unsigned)((r != r) ? 0 : (int)fmaxf(-127.0f, fminf(127.0f, r))) & 0xffu;
    }
    unsigned char *blk = row + (lane >> 2) * kQ8BlockBytes;
    if ((lane & 3) == 0) *reinterpret_cast<unsigned short *>(blk) = __half_as_ushort(__float2half_rn(d));
    unsigned short *dst = reinterpret_cast<unsigned short *>(blk + 2 + (lane & 3) * 8);
#pragma unroll
    for (int j = 0; j < 4; j++) dst[j] = (unsigned short)(q[2 * j] | (q[2 * j + 1] << 8));
}

// ---- q4_0 (crates/hipml-core/src/kv.rs:201-218): f16 scale + 16 bytes, byte j = value j (low
// nibble) | value j + 16 (high nibble); d = -vmax / 8 with vmax the element of largest
// magnitude (the first one on ties; NaN never wins; no element above zero leaves +0).
constexpr int kQ4BlockBytes = 18;

__device__ __forceinline__ size_t q4_row_offset(int kvh, int stride, int pos, int head_dim) {
    return ((size_t)kvh * (size_t)stride + (size_t)pos) * (size_t)(head_dim >> 5) *
           (size_t)kQ4BlockBytes;
}

// Of two candidates (magnitude, index, value) the one the definition's left fold keeps.
__device__ __forceinline__ void q4_pick(float &mag, int &idx, float &val, float omag, int oidx,
                                        float oval) {
    if (omag > mag || (omag == mag && oidx < idx)) {
        mag = omag;
        idx = oidx;
        val = oval;
    }
}

// The nibble of x for scale d (id = 1/d or 0): clamp(round-half-away(x * id) + 8, 0, 15), NaN -> 0.
__device__ __forceinline__ unsigned q4_code(float x, float id) {
    const float r = roundf(x * id) + 8.0f;
    return (r != r) ? 0u : (unsigned)fmaxf(0.0f, fminf(15.0f, r));
}

// One value per lane, a warp = one block.
__device__ __forceinline__ void q4_put(float x, int blk, int lane, unsigned char *row) {
    float mag = (x != x) ? -1.0f : fabsf(x), val = x;
    int idx = lane;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
        q4_pick(mag, idx, val, __shfl_xor_sync(0xffffffffu, mag, o), __shfl_xor_sync(0xffffffffu, idx, o),
                __shfl_xor_sync(0xffffffffu, val, o));
    const float vmax = mag > 0.0f ? val : 0.0f;
    const float d = -vmax / 8.0f;
    const float id = d != 0.0f ? 1.0f / d : 0.0f;
    const unsigned q = q4_code(x, id);
    const unsigned hi = __shfl_down_sync(0xffffffffu, q, 16);
    unsigned char *b = row + blk * kQ4BlockBytes;
    if (lane == 0) *reinterpret_cast<unsigned short *>(b) = __half_as_ushort(__float2half_rn(d));
    if (lane < 16) b[2 + lane] = (unsigned char)(q | (hi << 4));
}

// Eight values of one block held by one lane (lanes 4b..4b+3 share block b, values 8*(lane&3)..).
__device__ __forceinline__ void q4_put8(const float4 a, const float4 b, int lane, unsigned char *row) {
    const float x[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    float mag = -1.0f, val = 0.0f;
    int idx = 0;
#pragma unroll
    for (int j = 0; j < 8; j++)
        q4_pick(mag, idx, val, (x[j] != x[j]) ? -1.0f : fabsf(x[j]), (lane & 3) * 8 + j, x[j]);
#pragma unroll
    for (int o = 1; o <= 2; o <<= 1)
        q4_pick(mag, idx, val, __shfl_xor_sync(0xffffffffu, mag, o), __shfl_xor_sync(0xffffffffu, idx, o),
                __shfl_xor_sync(0xffffffffu, val, o));
    const float vmax = mag > 0.0f ? val : 0.0f;
    const float d = -vmax / 8.0f;
    const float id = d != 0.0f ? 1.0f / d : 0.0f;
    unsigned n = 0;   // this lane's eight nibbles
#pragma unroll
    for (int j = 0; j < 8; j++) n |= q4_code(x[j], id) << (4 * j);
    // lanes 0, 1 of the quad hold values 0..15 (low nibbles), lanes 2, 3 values 16..31 (high)
    const unsigned partner = __shfl_down_sync(0xffffffffu, n, 2);
    auto spread = [](unsigned h) {   // four nibbles -> four bytes
        h = (h | (h << 8)) & 0x00ff00ffu;
        return (h | (h << 4)) & 0x0f0f0f0fu;
    };
    unsigned char *blk = row + (lane >> 2) * kQ4BlockBytes;
    if ((lane & 3) == 0) *reinterpret_cast<unsigned short *>(blk) = __half_as_ushort(__float2half_rn(d));
    if ((lane & 3) < 2) {
        const unsigned lo = spread(n & 0xffffu) | (spread(partner & 0xffffu) << 4);
        const unsigned hi = spread(n >> 16) | (spread(partner >> 16) << 4);
        unsigned short *dst = reinterpret_cast<unsigned short *>(blk + 2 + (lane & 3) * 8);
        dst[0] = (unsigned short)lo;
        dst[1] = (unsigned short)(lo >> 16);
        dst[2] = (unsigned short)hi;
        dst[3] = (unsigned short)(hi >> 16);
    }
}

}  // namespace hipml
