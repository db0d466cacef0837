// Sequence-split decode across GPUs: the fold of a rank's split partials, the exchange of
// the folded (acc, max, sum) triples between the ranks and the final fold, in ONE kernel
// that talks to the peers through their memory (NVLink peer stores) instead of a collective
// call.
//
// Every rank owns a workspace that all ranks have mapped (peer access, IPC or symmetric
// memory): a header { epoch, CTA counter } and a double-buffered table
// cell[2][shards][n_heads][head_dim + 2] of 8-byte cells { value bits, epoch tag }. A call
// with epoch e (the local epoch + 1):
//   publish  each CTA folds its (head, 32 dims) of the local partials and stores every
//            result, paired with the tag e in ONE 8-byte store, into slot [e & 1][rank] of
//            EVERY rank's table (its own included). A cell is valid the moment its tag
//            reads e, so there is no fence, no flag and no second round trip: the exchange
//            costs one NVLink store latency.
//   collect  each CTA polls the cells of its (head, 32 dims) of every rank in its own table
//            until their tags read e (bounded polling: when the limit runs out it records
//            status 31 and leaves `out` alone), then folds the shards' triples into `out`.
// A rank can run at most one epoch ahead of a peer (its collect of epoch e needs the peer's
// publish of e, which comes after the peer's collect of e - 1), so two table slots are
// enough. The epoch lives in device memory and only grows (the last CTA of a call advances
// it), so a captured graph can be replayed. All ranks must make the same sequence of calls,
// and the workspace starts zero-filled (tag 0 is never a valid epoch).
//
// The algebra is the reference's split-K reduce (crates/hipml-kernels/kernels/
// attn_decode_kv.hip:491-532) applied twice; the reference itself is single-GPU.
#include "params.cuh"

namespace hipml {

namespace {

constexpr int kMaxShards = 16;
constexpr int kHeaderBytes = 256;   // int epoch, CTA counter

struct ExchangeParams {
    const float *acc;    // local partials [n_heads][splits][head_dim]
    const float *ml;     // [n_heads][splits][2]
    float *out;          // [n_heads][head_dim]
    int *status;
    int head_dim, splits, n_heads, shards, rank, phases;
    unsigned wait_polls;
    const int *len;      // optional: only min(splits, 64-key tiles of *len, run_cap) partials are live
    int run_cap;
    unsigned char *ws[kMaxShards];   // every rank's workspace as mapped in this process
};

// One 8-byte store / load, system scope, no ordering with other accesses needed: the tag
// travels with the value.
__device__ __forceinline__ void st_cell(uint2 *p, float value, int tag) {
    asm volatile("st.relaxed.sys.global.v2.b32 [%0], {%1, %2};" ::"l"(p), "r"(__float_as_uint(value)),
                 "r"(tag)
                 : "memory");
}
__device__ __forceinline__ uint2 ld_cell(const uint2 *p) {
    uint2 v;
    asm volatile("ld.relaxed.sys.global.v2.b32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ uint2 *cell_row(unsigned char *ws, int parity, int shards, int n_heads,
                                           int head_dim, int shard, int h) {
    uint2 *g = reinterpret_cast<uint2 *>(ws + kHeaderBytes);
    return g + (((size_t)parity * shards + shard) * n_heads + h) * (head_dim + 2);
}

// Polls one cell until its tag is e; false when the limit ran out.
__device__ __forceinline__ bool wait_cell(const uint2 *p, int e, unsigned polls, float &value) {
    for (unsigned i = 0; i < polls; i++) {
        const uint2 v = ld_cell(p);
        if ((int)v.y == e) {
            value = __uint_as_float(v.x);
            return true;
        }
        if (i > 16) __nanosleep(100);
    }
    return false;
}

// grid n_heads * head_dim / 32, block 256 (as attn_decode_fold).
__global__ void __launch_bounds__(256) attn_decode_fold_exchange(ExchangeParams p) {
    griddep_launch();
    griddep_wait();
    __shared__ float s_max[8];
    __shared__ float s_num[8][32];
    __shared__ float s_den[8];
    __shared__ float s_m[kMaxShards], s_l[kMaxShards];
    __shared__ int s_bad;
    const int chunks = p.head_dim >> 5;
    const int h = blockIdx.x / chunks, chunk = blockIdx.x - h * chunks;
    const int dl = threadIdx.x & 31, sg = threadIdx.x >> 5;
    int *hdr = reinterpret_cast<int *>(p.ws[p.rank]);
    // Every CTA reads the epoch before it adds itself to the counter, and the epoch advances
    // only after the last CTA has done so: all CTAs of a call see the same value.
    const int e = *reinterpret_cast<volatile int *>(hdr) + ((p.phases & 1) ? 1 : 0);
    const int parity = e & 1;
    if (threadIdx.x == 0) s_bad = 0;

    if (p.phases & 1) {
        // ---- publish: fold the local partials of (h, chunk) ...
        const float *pa = p.acc + (size_t)h * p.splits * p.head_dim + chunk * 32 + dl;
        const float *ml = p.ml + (size_t)h * p.splits * 2;
        const int nsplit = p.len ? min(min(p.splits, (*p.len + 63) >> 6), p.run_cap) : p.splits;
        float big = -INFINITY;
        for (int s = sg; s < nsplit; s += 8) big = fmaxf(big, ml[2 * s]);
        if (dl == 0) s_max[sg] = big;
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 8; i++) big = fmaxf(big, s_max[i]);
        float num = 0.0f, den = 0.0f;
        for (int s = sg; s < nsplit; s += 8) {
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
            // ... and store it, tagged, into every rank's table
            for (int w = 0; w < p.shards; w++) {
                uint2 *dst = cell_row(p.ws[w], parity, p.shards, p.n_heads, p.head_dim, p.rank, h);
                st_cell(dst + chunk * 32 + dl, n, e);
                if (chunk == 0 && dl == 0) {
                    st_cell(dst + p.head_dim, big, e);
                    st_cell(dst + p.head_dim + 1, d, e);
                }
            }
            if (dl == 0) {
                // epoch bookkeeping, off the critical path: the last CTA advances the epoch
                const int done = atomicAdd(hdr + 1, 1);
                if (done == (int)gridDim.x - 1) {
                    hdr[1] = 0;
                    *reinterpret_cast<volatile int *>(hdr) = e;
                }
            }
        }
    }

    if (p.phases & 2) {
        // ---- collect: warp sg takes shards sg, sg + 8; lane dl the cell of dim chunk*32 + dl
        __syncthreads();
        float num[2] = {0.0f, 0.0f};
        bool ok = true;
        for (int k = 0; k < 2; k++) {
            const int w = sg + 8 * k;
            if (w >= p.shards) break;
            const uint2 *src = cell_row(p.ws[p.rank], parity, p.shards, p.n_heads, p.head_dim, w, h);
            ok = wait_cell(src + chunk * 32 + dl, e, p.wait_polls, num[k]) && ok;
            if (dl < 2) {
                float v = 0.0f;
                ok = wait_cell(src + p.head_dim + dl, e, p.wait_polls, v) && ok;
                (dl == 0 ? s_m : s_l)[w] = v;
            }
        }
        if (!ok) s_bad = 1;
        __syncthreads();
        if (s_bad) {
            if (threadIdx.x == 0) atomicCAS(p.status, 0, 31);
        } else {
            float big = -INFINITY;
            for (int w = 0; w < p.shards; w++) big = fmaxf(big, s_m[w]);
            float part = 0.0f;
            for (int k = 0; k < 2; k++) {
                const int w = sg + 8 * k;
                if (w >= p.shards) break;
                const float wt = (s_m[w] == -INFINITY) ? 0.0f : exp2f(s_m[w] - big);
                part += num[k] * wt;
            }
            s_num[sg][dl] = part;
            __syncthreads();
            if (sg == 0) {
                float n = 0.0f, d = 0.0f;
#pragma unroll
                for (int i = 0; i < 8; i++) n += s_num[i][dl];
                for (int w = 0; w < p.shards; w++) {
                    const float wt = (s_m[w] == -INFINITY) ? 0.0f : exp2f(s_m[w] - big);
                    d += s_l[w] * wt;
                }
                p.out[(size_t)h * p.head_dim + chunk * 32 + dl] = d > 0.0f ? n / d : 0.0f;
            }
        }
    }
}

}  // namespace

size_t decode_exchange_bytes(int n_heads, int head_dim, int shards) {
    return (size_t)kHeaderBytes + 2 * (size_t)shards * n_heads * (head_dim + 2) * sizeof(uint2);
}

int launch_decode_fold_exchange(cudaStream_t stream, const float *part_acc, const float *part_ml,
                                float *out, int n_heads, int head_dim, int splits,
                                void *const *peer_ws, int shards, int rank, int phases,
                                unsigned wait_limit_us, int *status, const DecodeParams *live_runs) {
    ExchangeParams p;
    p.len = nullptr;
    p.run_cap = 0;
    if (live_runs && live_runs->run_cap > 0 && !live_runs->by_stride) {
        p.len = live_runs->len + live_runs->len_offset;
        p.run_cap = live_runs->run_cap;
    }
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
    p.wait_polls = wait_limit_us < 1 ? 16u : 16u + wait_limit_us * 4u;   // ~0.25 us per poll
    for (int w = 0; w < kMaxShards; w++)
        p.ws[w] = w < shards ? reinterpret_cast<unsigned char *>(peer_ws[w]) : nullptr;
    return launch_pdl(attn_decode_fold_exchange, dim3(n_heads * (head_dim >> 5)), dim3(256), 0, stream, 1, p);
}

}  // namespace hipml
