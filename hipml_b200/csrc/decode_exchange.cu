// Sequence-split decode across GPUs: the fold of a rank's split partials, the exchange of
// the folded (acc, max, sum) triples between the ranks and the final fold, in ONE kernel
// that talks to the peers through their memory (NVLink peer stores) instead of a collective
// call.
//
// Every rank owns a workspace that all ranks have mapped (peer access, IPC or symmetric
// memory): a header { epoch, CTA counter, flags[16] } and a double-buffered table
// gather[2][shards][n_heads][head_dim + 2]. A call with epoch e (the local epoch + 1):
//   publish  each CTA folds its (head, 32 dims) of the local partials and stores the result
//            into slot [e & 1][rank] of EVERY rank's table (its own included); the last CTA
//            to finish (counter) fences at system scope, stores e into flags[rank] of every
//            rank and advances the local epoch;
//   collect  each CTA waits until flags[w] >= e for every rank w of its own header (bounded
//            polling: when the limit runs out it records status 31 and leaves `out` alone),
//            then folds the shards' triples of its (head, 32 dims) into `out`.
// A rank can run at most one epoch ahead of a peer (its collect of epoch e needs the peer's
// publish of e, which comes after the peer's collect of e - 1), so two table slots are
// enough. The epochs live in device memory and only grow, so a captured graph can be
// replayed. All ranks must make the same sequence of calls.
//
// The algebra is the reference's split-K reduce (crates/hipml-kernels/kernels/
// attn_decode_kv.hip:491-532) applied twice; the reference itself is single-GPU.
#include "params.cuh"

namespace hipml {

namespace {

constexpr int kMaxShards = 16;
constexpr int kHeaderBytes = 256;   // int epoch, counter, pad[2], flags[16]

struct ExchangeParams {
    const float *acc;    // local partials [n_heads][splits][head_dim]
    const float *ml;     // [n_heads][splits][2]
    float *out;          // [n_heads][head_dim]
    int *status;
    int head_dim, splits, n_heads, shards, rank, phases;
    unsigned wait_polls;
    unsigned char *ws[kMaxShards];   // every rank's workspace as mapped in this process
};

__device__ __forceinline__ int ld_acquire_sys(const int *p) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_relaxed_sys(int *p, int v) {
    asm volatile("st.relaxed.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ float *gather_slot(unsigned char *ws, int parity, int shards, int n_heads,
                                              int head_dim, int shard, int h) {
    float *g = reinterpret_cast<float *>(ws + kHeaderBytes);
    return g + (((size_t)parity * shards + shard) * n_heads + h) * (head_dim + 2);
}

// grid n_heads * head_dim / 32, block 256 (as attn_decode_fold).
__global__ void __launch_bounds__(256) attn_decode_fold_exchange(ExchangeParams p) {
    __shared__ float s_max[8];
    __shared__ float s_num[8][32];
    __shared__ float s_den[8];
    __shared__ int s_ok;
    const int chunks = p.head_dim >> 5;
    const int h = blockIdx.x / chunks, chunk = blockIdx.x - h * chunks;
    const int dl = threadIdx.x & 31, sg = threadIdx.x >> 5;
    int *hdr = reinterpret_cast<int *>(p.ws[p.rank]);
    // Every CTA reads the epoch before it adds itself to the counter, and the epoch advances
    // only after the last CTA has done so: all CTAs of a call see the same value.
    const int e = *reinterpret_cast<volatile int *>(hdr) + ((p.phases & 1) ? 1 : 0);
    const int parity = e & 1;

    if (p.phases & 1) {
        // ---- publish: fold the local partials of (h, chunk) ...
        const float *pa = p.acc + (size_t)h * p.splits * p.head_dim + chunk * 32 + dl;
        const float *ml = p.ml + (size_t)h * p.splits * 2;
        float big = -INFINITY;
        for (int s = sg; s < p.splits; s += 8) big = fmaxf(big, ml[2 * s]);
        if (dl == 0) s_max[sg] = big;
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 8; i++) big = fmaxf(big, s_max[i]);
        float num = 0.0f, den = 0.0f;
        for (int s = sg; s < p.splits; s += 8) {
            const float m = ml[2 * s];
            const float w = (m == -INFINITY) ? 0.0f : exp2f(m - big);
            num += pa[(size_t)s * p.head_dim] * w;
            den += ml[2 * s + 1] * w;
        }
        s_num[sg][dl] = num;
        if (dl == 0) s_den[sg] = den;
        __syncthreads();
        if (sg == 0) {
            float n = 0.0f, d = 0.0f;
#pragma unroll
            for (int i = 0; i < 8; i++) {
                n += s_num[i][dl];
                d += s_den[i];
            }
            // ... and store it into every rank's table
            for (int w = 0; w < p.shards; w++) {
                float *dst = gather_slot(p.ws[w], parity, p.shards, p.n_heads, p.head_dim, p.rank, h);
                dst[chunk * 32 + dl] = n;
                if (chunk == 0 && dl == 0) {
                    dst[p.head_dim] = big;
                    dst[p.head_dim + 1] = d;
                }
            }
            __syncwarp();
            if (dl == 0) {
                __threadfence_system();
                const int done = atomicAdd(hdr + 1, 1);
                if (done == (int)gridDim.x - 1) {
                    // last CTA of this rank: everything of epoch e is on its way
                    // one system-scope fence orders all of it before the flags; the flag stores
                    // themselves are relaxed so that they leave back to back
                    __threadfence_system();
                    hdr[1] = 0;
                    for (int w = 0; w < p.shards; w++)
                        st_relaxed_sys(reinterpret_cast<int *>(p.ws[w]) + 4 + p.rank, e);
                    *reinterpret_cast<volatile int *>(hdr) = e;
                }
            }
        }
    }

    if (p.phases & 2) {
        // ---- collect: wait for every rank's epoch e (bounded), then fold the shards
        if (threadIdx.x == 0) s_ok = 1;
        __syncthreads();
        if (threadIdx.x < p.shards) {
            const int *flag = hdr + 4 + threadIdx.x;
            bool ok = false;
            for (unsigned i = 0; i < p.wait_polls; i++) {
                if (ld_acquire_sys(flag) - e >= 0) {
                    ok = true;
                    break;
                }
                __nanosleep(100);
            }
            if (!ok) {
                s_ok = 0;
                atomicCAS(p.status, 0, 31);
            }
        }
        __syncthreads();
        if (s_ok && sg == 0) {
            __threadfence_system();
            float big = -INFINITY;
            for (int w = 0; w < p.shards; w++) {
                const float *src = gather_slot(p.ws[p.rank], parity, p.shards, p.n_heads, p.head_dim, w, h);
                big = fmaxf(big, __ldcg(src + p.head_dim));
            }
            float num = 0.0f, den = 0.0f;
            for (int w = 0; w < p.shards; w++) {
                const float *src = gather_slot(p.ws[p.rank], parity, p.shards, p.n_heads, p.head_dim, w, h);
                const float m = __ldcg(src + p.head_dim);
                const float wt = (m == -INFINITY) ? 0.0f : exp2f(m - big);
                num += __ldcg(src + chunk * 32 + dl) * wt;
                den += __ldcg(src + p.head_dim + 1) * wt;
            }
            p.out[(size_t)h * p.head_dim + chunk * 32 + dl] = den > 0.0f ? num / den : 0.0f;
        }
    }
}

}  // namespace

size_t decode_exchange_bytes(int n_heads, int head_dim, int shards) {
    return (size_t)kHeaderBytes + 2 * (size_t)shards * n_heads * (head_dim + 2) * sizeof(float);
}

int launch_decode_fold_exchange(cudaStream_t stream, const float *part_acc, const float *part_ml,
                                float *out, int n_heads, int head_dim, int splits,
                                void *const *peer_ws, int shards, int rank, int phases,
                                unsigned wait_limit_us, int *status) {
    ExchangeParams p;
    p.acc = part_acc;
    p.ml = part_ml;
    p.out = out;
    p.status = status;
    p.head_dim = head_dim;
    p.splits = splits;
    p.n_heads = n_heads;
    p.shards = shards;
    p.rank = rank;
    p.phases = phases;
    p.wait_polls = wait_limit_us < 1 ? 1u : wait_limit_us * 4u;   // ~0.25 us per poll (sleep + load)
    for (int w = 0; w < kMaxShards; w++)
        p.ws[w] = w < shards ? reinterpret_cast<unsigned char *>(peer_ws[w]) : nullptr;
    attn_decode_fold_exchange<<<n_heads * (head_dim >> 5), 256, 0, stream>>>(p);
    return launch_status();
}

}  // namespace hipml
