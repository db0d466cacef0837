// Shared declarations for libhipml_cuda: error plumbing, the q8_0 geometry and
// small device helpers used by more than one kernel file.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>
#include <cstdlib>
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

// ---- programmatic dependent launch -----------------------------------------
// The path is a chain of short dependent kernels on one stream (append, split pass, fold;
// append, staging, chunk attention, combine), where the gap between a kernel's end and the
// start of the next costs as much as the small kernels themselves. Every kernel of this
// library therefore (1) lets the next launch of the stream be scheduled as soon as all of
// its own CTAs have started (griddep_launch at its top), and (2) waits for the previous
// grid to have completed and flushed before it touches memory (griddep_wait; anything
// before it is index arithmetic or loads of inputs that no kernel of the chain writes).
// Because every kernel waits before it writes, completion is transitive along the chain.
// Both instructions are no-ops in a launch without the attribute (a launch by name through
// hipml_module_launch_kernel, a kernel that follows a foreign kernel).
#ifdef __CUDACC__
__device__ __forceinline__ void griddep_launch() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void griddep_wait() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
}
#endif

// cudaLaunchKernelEx with the programmatic-stream-serialization attribute (and, for
// cluster_x > 1, the cluster dimension).
template <typename... KArgs, typename... Args>
int launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
               unsigned cluster_x, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.numAttrs = 1;
    if (cluster_x > 1) {
        attr[1].id = cudaLaunchAttributeClusterDimension;
        attr[1].val.clusterDim.x = cluster_x;
        attr[1].val.clusterDim.y = 1;
        attr[1].val.clusterDim.z = 1;
        cfg.numAttrs = 2;
    }
    cfg.attrs = attr;
    return static_cast<int>(cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...));
}

// The same for a kernel given by address with an argument array (the kernels that keep the
// reference's parameter lists).
inline int launch_pdl_args(const void *kernel, dim3 grid, dim3 block, void **args, size_t smem,
                           cudaStream_t stream) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    return static_cast<int>(cudaLaunchKernelExC(&cfg, kernel, args));
}

// Host-side addresses of the kernels that keep the reference's entry names and
// parameter lists (one lookup per defining file); nullptr when the name is not there.
const void *lookup_kv_kernel(const char *name);
const void *lookup_decode_kernel(const char *name);
const void *lookup_chunk_kernel(const char *name);
const void *lookup_cols_kernel(const char *name);
const void *lookup_front_kernel(const char *name);

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
