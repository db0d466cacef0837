// Shared declarations for libhipml_cuda: error plumbing, the q8_0 geometry and
// small device helpers used by more than one kernel file.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>
#include <cstring>

#include "../../include/hipml_cuda.h"

namespace hipml {

// q8_0: f16 scale + 32 int8 codes (crates/hipml-core/src/kv.rs:11-14).
constexpr int kBlock = 32;
constexpr int kQ8BlockBytes = 34;

// Records the sentence for hipml_last_error_message() and returns `code`.
int fail(int code, const char *fmt, ...);

inline cudaStream_t as_stream(hipml_stream_t s) { return reinterpret_cast<cudaStream_t>(s); }

// Launch check: cudaGetLastError after a <<<>>> launch, as an int for the C ABI.
inline int launch_status() { return static_cast<int>(cudaGetLastError()); }

// Host-side addresses of the kernels that keep the reference's entry names and
// parameter lists (one lookup per defining file); nullptr when the name is not there.
const void *lookup_kv_kernel(const char *name);
const void *lookup_decode_kernel(const char *name);
const void *lookup_chunk_kernel(const char *name);
const void *lookup_cols_kernel(const char *name);

// Device status word set by kernels whose bounded waits ran out.
int *device_status_word();

// ---- device helpers -------------------------------------------------------

// Byte offset of row (kvh, pos) of a head-major q8 cache with `stride` rows per head.
__device__ __forceinline__ size_t q8_row_offset(int kvh, int stride, int pos, int head_dim) {
    return ((size_t)kvh * (size_t)stride + (size_t)pos) * (size_t)(head_dim >> 5) *
           (size_t)kQ8BlockBytes;
}

__device__ __forceinline__ float half_bits_to_float(uint16_t h) {
    return __half2float(__ushort_as_half(h));
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

}  // namespace hipml
