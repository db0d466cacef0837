// Sequence-split decode across GPUs: every rank folds its own cache rows to one
// (acc, max, sum) triple per head, the triples travel between the ranks, and every rank
// folds all of them. The exchange runs INSIDE the decode kernels, through the peers' memory
// (NVLink peer stores), not as a collective call.
//
// Every rank owns a workspace that all ranks have mapped (peer access, IPC or symmetric
// memory): a 256-byte header { epoch, arrival counter } and a double-buffered table
// cell[2][shards][n_heads][head_dim + 2] of 8-byte cells { value bits, epoch tag }. A call
// with epoch e (the local epoch + 1):
//   publish  the CTA of the split pass that holds a KV head's final fold (decode_fold.cuh,
//            attn_decode_tc.cu) stores every value of its heads' triples, paired with the tag
//            e in ONE 64-bit store, into slot [e & 1][rank] of EVERY rank's table (its own
//            included). A cell is valid the moment its tag reads e, so there is no fence, no
//            flag and no second round trip: the exchange costs one NVLink store latency.
//   collect  the same CTA (or the collect launch below, for callers that split the two
//            halves) polls the cells of its heads of every rank in its own table until their
//            tags read e (bounded by time: when the limit runs out it records status 31 and
//            leaves `out` alone), then folds the ranks' triples into `out`.
// A rank can run at most one epoch ahead of a peer (its collect of epoch e needs the peer's
// publish of e, which comes after the peer's collect of e - 1), so two table slots are
// enough. The epoch lives in device memory and only grows (the last publishing CTA of a call
// advances it), so a captured graph can be replayed. All ranks must make the same sequence
// of calls, and the workspace starts zero-filled (tag 0 is never a valid epoch). If one rank
// skips a call (a host-side error before its launch) the epochs drift apart for good: every
// later collect times out with status 31 until all ranks zero their workspaces again between
// steps (hipml_memset of the whole workspace on every rank, then a host barrier).
//
// The algebra is the reference's split-K reduce (crates/hipml-kernels/kernels/
// attn_decode_kv.hip:491-532) applied twice; the reference itself is single-GPU.
#include "decode_fold.cuh"

namespace hipml {

namespace {

// grid ceil(n_heads / 8), block 256: warp = head.
__global__ void __launch_bounds__(256) attn_decode_collect(DecodeParams p, int *status) {
    griddep_launch();
    griddep_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int h = blockIdx.x * 8 + warp;
    if (h >= p.n_heads) return;
    if (p.xch.by_head && exchange_owner(p.xch, p.n_heads, h) != p.xch.rank) return;
    const int e = *reinterpret_cast<volatile int *>(p.xch.ws[p.xch.rank]);
    const unsigned long long deadline = global_timer_ns() + 1000ull * p.xch.wait_us;
    FoldAcc f;
    if (exchange_collect_warp(p.xch, p.n_heads, h, e, deadline, lane, f))
        fold_emit(p, 0, h, f, lane, true);
    else if (lane == 0)
        atomicCAS(status, 0, 31);
}

// The exchange as a launch of its own, for many ranks: one SM cannot feed NVLink with the
// triples of six heads for eight peers (100 KB of 16-byte stores took ~10 us from one SM), so
// with more than kInKernelShards ranks the split pass leaves its folded triples in the local
// staging area of the workspace and this grid of (n_heads, shards) CTAs moves them: CTA (h, w)
// stores head h's triple into rank w's table; CTA (h, 0) then collects head h (warp = rank).
// grid (n_heads, shards), block 256.
__global__ void __launch_bounds__(256) attn_decode_exchange_wide(DecodeParams p, int *status) {
    griddep_launch();
    griddep_wait();
    __shared__ float s_m[16], s_l[16];
    __shared__ float s_part[8][256];
    __shared__ int s_bad;
    const int h = blockIdx.x, w = blockIdx.y;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    int *hdr = reinterpret_cast<int *>(p.xch.ws[p.xch.rank]);
    // every CTA reads the epoch before it adds itself to the counter; the last one advances it
    const int e = *reinterpret_cast<volatile int *>(hdr) + 1;
    const float *stage = reinterpret_cast<const float *>(
        p.xch.ws[p.xch.rank] + kExchangeHeaderBytes +
        2 * (size_t)p.xch.shards * p.n_heads * 258 * 8) + (size_t)h * 258;
    {
        unsigned long long *row = cell_row(p.xch.ws[w], e & 1, p.xch.shards, p.n_heads, p.xch.rank, h);
        st_cell(row + tid, stage[tid], e);
        if (tid < 2) st_cell(row + 256 + tid, stage[256 + tid], e);
    }
    if (tid == 0) s_bad = 0;
    __syncthreads();
    if (tid == 0) {
        const int total = (int)(gridDim.x * gridDim.y);
        if (atomicAdd(hdr + 1, 1) == total - 1) {
            hdr[1] = 0;
            *reinterpret_cast<volatile int *>(hdr) = e;
        }
    }
    if (w != 0) return;
    // ---- collect head h: warp r (and r + 8) polls rank r's cells, eight per lane
    const unsigned long long deadline = global_timer_ns() + 1000ull * p.xch.wait_us;
    bool ok = true;
    float vals[2][8];
    for (int k = 0; k < 2; k++) {
        const int r = warp + 8 * k;
        if (r >= p.xch.shards) break;
        const unsigned long long *src = cell_row(p.xch.ws[p.xch.rank], e & 1, p.xch.shards, p.n_heads, r, h);
        unsigned long long c[8];
        for (unsigned i = 0;; i++) {
            ld_cell2(src + lane * 8, c[0], c[1]);
            ld_cell2(src + lane * 8 + 2, c[2], c[3]);
            ld_cell2(src + lane * 8 + 4, c[4], c[5]);
            ld_cell2(src + lane * 8 + 6, c[6], c[7]);
            bool all = true;
#pragma unroll
            for (int j = 0; j < 8; j++) all = all && (int)(c[j] >> 32) == e;
            if (lane == 0) {
                unsigned long long a, b;
                ld_cell2(src + 256, a, b);
                all = all && (int)(a >> 32) == e && (int)(b >> 32) == e;
                if (all) {
                    s_m[r] = __uint_as_float((unsigned)a);
                    s_l[r] = __uint_as_float((unsigned)b);
                }
            }
            if (__all_sync(0xffffffffu, all)) break;
            if ((i & 7) == 7) {
                if (global_timer_ns() > deadline) {
                    ok = false;
                    break;
                }
                __nanosleep(64);
            }
        }
        if (!ok) break;
#pragma unroll
        for (int j = 0; j < 8; j++) vals[k][j] = __uint_as_float((unsigned)c[j]);
    }
    if (!ok) s_bad = 1;
    __syncthreads();
    if (s_bad) {
        if (tid == 0) atomicCAS(status, 0, 31);
        return;
    }
    float big = -INFINITY;
    for (int r = 0; r < p.xch.shards; r++) big = fmaxf(big, s_m[r]);
    // weighted rows to shared memory, then the sum in rank order (as the other forms do)
    for (int k = 0; k < 2; k++) {
        const int r = warp + 8 * k;
        if (r >= p.xch.shards) break;
        const float wt = (s_m[r] == -INFINITY) ? 0.0f : exp2f(s_m[r] - big);
#pragma unroll
        for (int j = 0; j < 8; j++) vals[k][j] = __fmul_rn(vals[k][j], wt);
    }
    float out = 0.0f;
    for (int k = 0; k < 2; k++) {
        if (8 * k >= p.xch.shards) break;
        __syncthreads();
        if (warp + 8 * k < p.xch.shards) {
#pragma unroll
            for (int j = 0; j < 8; j++) s_part[warp][lane * 8 + j] = vals[k][j];
        }
        __syncthreads();
        for (int r = 0; r < 8 && 8 * k + r < p.xch.shards; r++) out = __fadd_rn(out, s_part[r][tid]);
    }
    float den = 0.0f;
    for (int r = 0; r < p.xch.shards; r++) {
        const float wt = (s_m[r] == -INFINITY) ? 0.0f : exp2f(s_m[r] - big);
        den = __fadd_rn(den, __fmul_rn(s_l[r], wt));
    }
    p.out[(size_t)h * p.out_head_stride + tid] = den > 0.0f ? __fdiv_rn(out, den) : 0.0f;
}

}  // namespace

size_t decode_exchange_bytes(int n_heads, int head_dim, int shards) {
    // header, the double-buffered table of cells, and the local staging rows of the wide form
    return (size_t)kExchangeHeaderBytes + 2 * (size_t)shards * n_heads * (head_dim + 2) * 8 +
           (size_t)n_heads * (head_dim + 2) * 4;
}

float *decode_exchange_stage(void *ws, int n_heads, int shards) {
    return reinterpret_cast<float *>(reinterpret_cast<unsigned char *>(ws) + kExchangeHeaderBytes +
                                     2 * (size_t)shards * n_heads * 258 * 8);
}

int launch_decode_exchange_wide(cudaStream_t stream, const DecodeParams &p, int *status) {
    return launch_pdl(attn_decode_exchange_wide, dim3(p.n_heads, p.xch.shards), dim3(256), 0, stream, 1, p,
                      status);
}

int launch_decode_collect(cudaStream_t stream, const DecodeParams &p, int *status) {
    return launch_pdl(attn_decode_collect, dim3((p.n_heads + 7) / 8), dim3(256), 0, stream, 1, p, status);
}

}  // namespace hipml
