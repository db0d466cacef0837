// KV append for the full-attention layers: q8_0 quantise-and-append (one row,
// a block of rows, one row per slot) and the plain f32 append.
//
// Format definition: crates/hipml-core/src/kv.rs:187-200 (quantize_block, Q8
// arm). Per 32-value block: amax = max|x|, d = amax/127 (f32), id = 1/d from
// that f32 d (0 if d == 0), scale = f16(d) round-to-nearest-even, code =
// clamp(round-half-away(x*id), -127, 127). The bytes written here are
// bit-identical to the host encode; the kernels this file replaces are
// crates/hipml-kernels/kernels/kv_encode.hip:64-98,111-148,246-284 and
// kv_append_f32.hip:10-26, attn_chunk_f32.hip:100-119.
//
// Shape of the work: a CTA of head_dim threads (one warp per 32-value block)
// quantises one K row and one V row of one KV head into shared memory, then
// streams each finished 272-byte row to the cache with 16-byte stores, so the
// cache sees whole-sector writes instead of one byte per lane.
#include "common.cuh"
#include "q8_pack.cuh"

namespace hipml {

namespace {


// Quantise x (this lane's value of block `blk`) into row image `row`.
__device__ __forceinline__ void q8_put(float x, int blk, int lane, unsigned char *row) {
    // max from 0 that ignores NaN operands, as the host definition's fold does
    const float amax = fmaxf(0.0f, warp_max(fabsf(x)));
    const float d = amax / 127.0f;
    const float id = d > 0.0f ? 1.0f / d : 0.0f;
    const float r = roundf(x * id);
    // A NaN input encodes as 0, as the host definition's `as i8` does.
    const int q = (r != r) ? 0 : (int)fmaxf(-127.0f, fminf(127.0f, r));
    unsigned char *b = row + blk * kQ8BlockBytes;
    if (lane == 0) *reinterpret_cast<unsigned short *>(b) = __half_as_ushort(__float2half_rn(d));
    b[2 + lane] = (unsigned char)(signed char)q;
}

// One (K row, V row) pair of one KV head. All threads of the CTA must call it.
template <bool kQ4 = false>
__device__ __forceinline__ void encode_pair(const float *ksrc, const float *vsrc,
                                            unsigned char *kdst, unsigned char *vdst,
                                            int head_dim, unsigned char *krow,
                                            unsigned char *vrow) {
    const int tid = threadIdx.x;
    const int blk = tid >> 5, lane = tid & 31;
    if (tid < head_dim) {
        if constexpr (kQ4) {
            q4_put(ksrc[tid], blk, lane, krow);
            q4_put(vsrc[tid], blk, lane, vrow);
        } else {
            q8_put(ksrc[tid], blk, lane, krow);
            q8_put(vsrc[tid], blk, lane, vrow);
        }
    }
    __syncthreads();
    const int row_bytes = (head_dim >> 5) * (kQ4 ? kQ4BlockBytes : kQ8BlockBytes);
    row_store(kdst, krow, row_bytes, tid, blockDim.x);
    row_store(vdst, vrow, row_bytes, tid, blockDim.x);
    __syncthreads();
}

}  // namespace

// Entry names and parameter lists are the reference's, so a launch by name
// with its argument array works unchanged (grid (n_kv), block head_dim).
extern "C" __global__ void kv_encode_q8(const float *__restrict__ k, const float *__restrict__ v,
                                        unsigned char *__restrict__ kc,
                                        unsigned char *__restrict__ vc, int head_dim, int stride,
                                        const int *__restrict__ step) {
    griddep_launch();
    griddep_wait();
    __shared__ __align__(16) unsigned char krow[kMaxRowBytes];
    __shared__ __align__(16) unsigned char vrow[kMaxRowBytes];
    const int h = blockIdx.x;
    const size_t off = q8_row_offset(h, stride, step[0], head_dim);
    encode_pair(k + (size_t)h * head_dim, v + (size_t)h * head_dim, kc + off, vc + off, head_dim,
                krow, vrow);
}

// grid: any count up to n_kv*rows (the reference launches exactly n_kv*rows);
// the CTA walks (row, head) pairs with a grid stride.
extern "C" __global__ void kv_encode_bulk_q8(const float *__restrict__ k,
                                             const float *__restrict__ v,
                                             unsigned char *__restrict__ kc,
                                             unsigned char *__restrict__ vc, int n_kv,
                                             int head_dim, int stride, int start, int rows,
                                             int src0) {
    griddep_launch();
    griddep_wait();
    __shared__ __align__(16) unsigned char krow[kMaxRowBytes];
    __shared__ __align__(16) unsigned char vrow[kMaxRowBytes];
    const long long total = (long long)n_kv * rows;
    for (long long idx = blockIdx.x; idx < total; idx += gridDim.x) {
        const int r = (int)(idx / n_kv);
        const int h = (int)(idx - (long long)r * n_kv);
        const size_t src = ((size_t)(src0 + r) * n_kv + h) * (size_t)head_dim;
        const size_t off = q8_row_offset(h, stride, start + r, head_dim);
        encode_pair(k + src, v + src, kc + off, vc + off, head_dim, krow, vrow);
    }
}

// The throughput form of the bulk append for head_dim 256 and 16-byte-aligned sources
// (what hipml_kv_encode_bulk launches; the kernel above keeps the reference's launch shape
// for launches by name). One warp per (row, KV head): a lane loads 8 consecutive values of
// the K row and of the V row (four 16-byte loads in flight), four lanes agree on a block's
// maximum with two shuffles, the 272-byte images are assembled in shared memory and leave
// as 16-byte stores. grid = ceil(n_kv*rows / 8), block 256. Same arithmetic per value as
// q8_put, so the bytes are identical.
__global__ void __launch_bounds__(256) kv_encode_bulk_q8_w(const float *__restrict__ k,
                                                           const float *__restrict__ v,
                                                           unsigned char *__restrict__ kc,
                                                           unsigned char *__restrict__ vc, int n_kv,
                                                           int stride, int start, int rows,
                                                           int src0) {
    __shared__ __align__(16) unsigned char img[8][2][kMaxRowBytes];
    griddep_launch();
    griddep_wait();   // the f32 rows may come from a grid that is still running
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long idx = (long long)blockIdx.x * 8 + warp;
    if (idx >= (long long)n_kv * rows) return;
    const int r = (int)(idx / n_kv);
    const int h = (int)(idx - (long long)r * n_kv);
    const size_t src = ((size_t)(src0 + r) * n_kv + h) * 256 + (size_t)lane * 8;
    const float4 ka = __ldg(reinterpret_cast<const float4 *>(k + src));
    const float4 kb = __ldg(reinterpret_cast<const float4 *>(k + src) + 1);
    const float4 va = __ldg(reinterpret_cast<const float4 *>(v + src));
    const float4 vb = __ldg(reinterpret_cast<const float4 *>(v + src) + 1);
    q8_put8(ka, kb, lane, img[warp][0]);
    q8_put8(va, vb, lane, img[warp][1]);
    __syncwarp();
    const size_t off = q8_row_offset(h, stride, start + r, 256);
    row_store(kc + off, img[warp][0], kMaxRowBytes, lane, 32);
    row_store(vc + off, img[warp][1], kMaxRowBytes, lane, 32);
}

int launch_kv_encode_bulk_rows(cudaStream_t stream, const float *k, const float *v,
                               unsigned char *kc, unsigned char *vc, int n_kv, int stride,
                               int start, int src0, int rows) {
    const long long pairs = (long long)n_kv * rows;
    return launch_pdl(kv_encode_bulk_q8_w, dim3((unsigned)((pairs + 7) / 8)), dim3(256), 0, stream, 1, k, v,
                      kc, vc, n_kv, stride, start, rows, src0);
}

// grid (n_kv, slots): slot s appends its row at pos[2*s] in the cache at s*slot_bytes.
extern "C" __global__ void kv_encode_q8_b(const float *__restrict__ k, const float *__restrict__ v,
                                          unsigned char *__restrict__ kc,
                                          unsigned char *__restrict__ vc, int n_kv, int head_dim,
                                          int stride, const int *__restrict__ pos,
                                          int slot_bytes) {
    griddep_launch();
    griddep_wait();
    __shared__ __align__(16) unsigned char krow[kMaxRowBytes];
    __shared__ __align__(16) unsigned char vrow[kMaxRowBytes];
    const int h = blockIdx.x, slot = blockIdx.y;
    const size_t src = ((size_t)slot * n_kv + h) * (size_t)head_dim;
    const size_t off =
        (size_t)slot * (size_t)slot_bytes + q8_row_offset(h, stride, pos[slot * 2], head_dim);
    encode_pair(k + src, v + src, kc + off, vc + off, head_dim, krow, vrow);
}

// ---- q4_0 forms of the three entries (crates/hipml-kernels/kernels/kv_encode.hip:150-238,
// 286-320): same parameter lists and launch shapes, 18-byte blocks.
extern "C" __global__ void kv_encode_q4(const float *__restrict__ k, const float *__restrict__ v,
                                        unsigned char *__restrict__ kc,
                                        unsigned char *__restrict__ vc, int head_dim, int stride,
                                        const int *__restrict__ step) {
    griddep_launch();
    griddep_wait();
    __shared__ __align__(16) unsigned char krow[kMaxRowBytes];
    __shared__ __align__(16) unsigned char vrow[kMaxRowBytes];
    const int h = blockIdx.x;
    const size_t off = q4_row_offset(h, stride, step[0], head_dim);
    encode_pair<true>(k + (size_t)h * head_dim, v + (size_t)h * head_dim, kc + off, vc + off, head_dim,
                      krow, vrow);
}

extern "C" __global__ void kv_encode_bulk_q4(const float *__restrict__ k,
                                             const float *__restrict__ v,
                                             unsigned char *__restrict__ kc,
                                             unsigned char *__restrict__ vc, int n_kv,
                                             int head_dim, int stride, int start, int rows,
                                             int src0) {
    griddep_launch();
    griddep_wait();
    __shared__ __align__(16) unsigned char krow[kMaxRowBytes];
    __shared__ __align__(16) unsigned char vrow[kMaxRowBytes];
    const long long total = (long long)n_kv * rows;
    for (long long idx = blockIdx.x; idx < total; idx += gridDim.x) {
        const int r = (int)(idx / n_kv);
        const int h = (int)(idx - (long long)r * n_kv);
        const size_t src = ((size_t)(src0 + r) * n_kv + h) * (size_t)head_dim;
        const size_t off = q4_row_offset(h, stride, start + r, head_dim);
        encode_pair<true>(k + src, v + src, kc + off, vc + off, head_dim, krow, vrow);
    }
}

extern "C" __global__ void kv_encode_q4_b(const float *__restrict__ k, const float *__restrict__ v,
                                          unsigned char *__restrict__ kc,
                                          unsigned char *__restrict__ vc, int n_kv, int head_dim,
                                          int stride, const int *__restrict__ pos,
                                          int slot_bytes) {
    griddep_launch();
    griddep_wait();
    __shared__ __align__(16) unsigned char krow[kMaxRowBytes];
    __shared__ __align__(16) unsigned char vrow[kMaxRowBytes];
    const int h = blockIdx.x, slot = blockIdx.y;
    const size_t src = ((size_t)slot * n_kv + h) * (size_t)head_dim;
    const size_t off =
        (size_t)slot * (size_t)slot_bytes + q4_row_offset(h, stride, pos[slot * 2], head_dim);
    encode_pair<true>(k + src, v + src, kc + off, vc + off, head_dim, krow, vrow);
}

// Throughput form of the q4_0 bulk append (head_dim 256, 16-byte-aligned sources): one warp
// per (row, KV head), as kv_encode_bulk_q8_w.
__global__ void __launch_bounds__(256) kv_encode_bulk_q4_w(const float *__restrict__ k,
                                                           const float *__restrict__ v,
                                                           unsigned char *__restrict__ kc,
                                                           unsigned char *__restrict__ vc, int n_kv,
                                                           int stride, int start, int rows,
                                                           int src0) {
    __shared__ __align__(16) unsigned char img[8][2][8 * kQ4BlockBytes];
    griddep_launch();
    griddep_wait();   // the f32 rows may come from a grid that is still running
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long idx = (long long)blockIdx.x * 8 + warp;
    if (idx >= (long long)n_kv * rows) return;
    const int r = (int)(idx / n_kv);
    const int h = (int)(idx - (long long)r * n_kv);
    const size_t src = ((size_t)(src0 + r) * n_kv + h) * 256 + (size_t)lane * 8;
    const float4 ka = __ldg(reinterpret_cast<const float4 *>(k + src));
    const float4 kb = __ldg(reinterpret_cast<const float4 *>(k + src) + 1);
    const float4 va = __ldg(reinterpret_cast<const float4 *>(v + src));
    const float4 vb = __ldg(reinterpret_cast<const float4 *>(v + src) + 1);
    q4_put8(ka, kb, lane, img[warp][0]);
    q4_put8(va, vb, lane, img[warp][1]);
    __syncwarp();
    const size_t off = q4_row_offset(h, stride, start + r, 256);
    row_store(kc + off, img[warp][0], 8 * kQ4BlockBytes, lane, 32);
    row_store(vc + off, img[warp][1], 8 * kQ4BlockBytes, lane, 32);
}

int launch_kv_encode_bulk_rows_q4(cudaStream_t stream, const float *k, const float *v,
                                  unsigned char *kc, unsigned char *vc, int n_kv, int stride,
                                  int start, int src0, int rows) {
    const long long pairs = (long long)n_kv * rows;
    return launch_pdl(kv_encode_bulk_q4_w, dim3((unsigned)((pairs + 7) / 8)), dim3(256), 0, stream, 1, k, v,
                      kc, vc, n_kv, stride, start, rows, src0);
}

// One token's K and V rows into row step[0] of the position-major f32 caches. The entry name,
// parameter list and launch shape (ceil(2 * width / 256) blocks of 256 threads, one element per
// thread) are what a launch by name passes (AttnLayer::append_at, crates/hipml-kernels/src/
// attn_gpu.rs:885-912); the body treats the launch as one index space over the pair of rows.
extern "C" __global__ void kv_append_f32(float *__restrict__ k_cache, float *__restrict__ v_cache,
                                         const float *__restrict__ k, const float *__restrict__ v,
                                         const int *__restrict__ step, int width) {
    griddep_launch();
    griddep_wait();
    const int e = blockIdx.x * blockDim.x + threadIdx.x;   // element of the (K row | V row) pair
    const int which = e / width, col = e - which * width;
    if (which > 1) return;
    float *cache = which ? v_cache : k_cache;
    const float *row = which ? v : k;
    cache[(size_t)step[0] * (size_t)width + col] = row[col];
}

// Rows t < tokens of k/v land at cache row pos0+t. One thread per 4 floats when
// width is a multiple of 4 (it is 1024 on the shipped shape), else per float.
extern "C" __global__ void kv_append_chunk_f32(float *__restrict__ k_cache,
                                               float *__restrict__ v_cache,
                                               const float *__restrict__ k,
                                               const float *__restrict__ v, int pos0, int width,
                                               int tokens) {
    griddep_launch();
    griddep_wait();
    const size_t n = (size_t)tokens * (size_t)width;
    const size_t base = (size_t)pos0 * (size_t)width;
    const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t nthreads = (size_t)gridDim.x * blockDim.x;
    const bool vec = (width % 4 == 0) &&
                     (((reinterpret_cast<size_t>(k_cache) | reinterpret_cast<size_t>(v_cache) |
                        reinterpret_cast<size_t>(k) | reinterpret_cast<size_t>(v)) & 15) == 0);
    if (vec) {
        const size_t n4 = n / 4;
        float4 *kd = reinterpret_cast<float4 *>(k_cache + base);
        float4 *vd = reinterpret_cast<float4 *>(v_cache + base);
        for (size_t i = tid; i < n4; i += nthreads) {
            kd[i] = reinterpret_cast<const float4 *>(k)[i];
            vd[i] = reinterpret_cast<const float4 *>(v)[i];
        }
    } else {
        for (size_t i = tid; i < n; i += nthreads) {
            k_cache[base + i] = k[i];
            v_cache[base + i] = v[i];
        }
    }
}

const void *lookup_kv_kernel(const char *name) {
    if (strcmp(name, "kv_encode_q8") == 0) return (const void *)kv_encode_q8;
    if (strcmp(name, "kv_encode_bulk_q8") == 0) return (const void *)kv_encode_bulk_q8;
    if (strcmp(name, "kv_encode_q8_b") == 0) return (const void *)kv_encode_q8_b;
    if (strcmp(name, "kv_encode_q4") == 0) return (const void *)kv_encode_q4;
    if (strcmp(name, "kv_encode_bulk_q4") == 0) return (const void *)kv_encode_bulk_q4;
    if (strcmp(name, "kv_encode_q4_b") == 0) return (const void *)kv_encode_q4_b;
    if (strcmp(name, "kv_append_f32") == 0) return (const void *)kv_append_f32;
    if (strcmp(name, "kv_append_chunk_f32") == 0) return (const void *)kv_append_chunk_f32;
    return nullptr;
}

}  // namespace hipml
