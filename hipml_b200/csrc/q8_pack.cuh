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

}  // namespace hipml
