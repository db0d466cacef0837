// hipml_attn_decode_kv_static: the single-stream q8 decode for callers that cannot allocate.
//
// hipml_attn_decode_kv needs two caller-owned scratch buffers for the split partials. Some
// callers have no way to provide them: a host that embeds the library behind a fixed-size
// arena and is not allowed to call cudaMalloc once it is serving, a thin language binding
// that can pass its tensors but has no device allocator of its own, a latency-critical loop
// that must not touch the allocator (an allocation can synchronise the device). For them this
// entry keeps the partials in a file-scope device array that lives in the library image: every
// GPU that loads the library holds those 6.05 MiB until the process exits.
//
// What that implies for the caller:
//  * the array is sized for n_heads * splits * (head_dim + 2) <= kMaxScratchFloats floats
//    (24 heads x 256 splits x 258); larger requests are rejected, nothing is launched;
//  * the first call on each device resolves the array's device address (cudaGetSymbolAddress
//    with that device current); make that first call outside any stream capture;
//  * every call uses the same array and finds the previous call's partials in it. Nothing
//    has to be cleared: the split pass writes every (head, split) slot it later folds. But two
//    calls that overlap on the GPU (different streams, or graphs replayed concurrently)
//    would write the same slots, so calls must be ordered on the device.
#include "params.cuh"

namespace hipml {

namespace {

constexpr size_t kMaxScratchFloats = (size_t)24 * 256 * (256 + 2);

// Split partials: part_acc [n_heads][splits][head_dim] followed by part_ml [n_heads][splits][2].
static __device__ __align__(256) float g_decode_scratch[kMaxScratchFloats];

// The symbol above is a host-side handle, not a device pointer: its device address has to
// be asked for, once per device, with that device current.
float *scratch_address(int *status) {
    static float *cached[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) {
        *status = (int)e;
        return nullptr;
    }
    if (dev < 0 || dev >= 64) {
        *status = fail(HIPML_ERR_INVALID_ARGUMENT, "device ordinal %d is out of range", dev);
        return nullptr;
    }
    if (!cached[dev]) {
        float *ptr = nullptr;
        e = cudaGetSymbolAddress(reinterpret_cast<void **>(&ptr), g_decode_scratch);
        if (e != cudaSuccess) {
            *status = (int)e;
            return nullptr;
        }
        cached[dev] = ptr;
    }
    *status = 0;
    return cached[dev];
}

}  // namespace

}  // namespace hipml

using namespace hipml;

extern "C" int hipml_attn_decode_kv_static(hipml_stream_t stream, const int *step, int selector,
                                           const float *q, const void *k, const void *v,
                                           float *out, int n_heads, int n_kv, int head_dim,
                                           int stride, float scale, int splits, size_t k_off,
                                           size_t v_off) {
    if (splits < 1) splits = 1;
    if (n_heads <= 0 || head_dim <= 0)
        return fail(HIPML_ERR_INVALID_ARGUMENT, "n_heads %d / head_dim %d must be positive",
                    n_heads, head_dim);
    const size_t need = (size_t)n_heads * splits * ((size_t)head_dim + 2);
    if (need > kMaxScratchFloats)
        return fail(HIPML_ERR_WORKSPACE,
                    "static decode scratch: n_heads %d x splits %d x (head_dim %d + 2) = %zu floats "
                    "exceeds the built-in %zu; use hipml_attn_decode_kv with caller scratch",
                    n_heads, splits, head_dim, need, kMaxScratchFloats);
    int status = 0;
    float *scratch = scratch_address(&status);
    if (!scratch) return status;
    float *part_acc = scratch;
    float *part_ml = scratch + (size_t)n_heads * splits * head_dim;
    return hipml_attn_decode_kv(stream, step, selector, q, k, v, part_acc, part_ml, out, n_heads,
                                n_kv, head_dim, stride, scale, splits, k_off, v_off);
}
