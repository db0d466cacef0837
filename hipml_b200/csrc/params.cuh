// Parameter blocks and host-side launch helpers shared between the kernel files and
// the C-ABI launchers.
#pragma once

#include "common.cuh"

namespace hipml {

// Split-K decode over the q8_0 cache (attn_decode.cu).
struct DecodeParams {
    const float *q;
    const unsigned char *k;
    const unsigned char *v;
    float *part_acc;
    float *part_ml;
    const int *len;       // live length of slot s is len[s*len_stride + len_offset]
    int len_stride;
    int len_offset;
    int n_heads, n_kv, head_dim, stride;
    float scale_log2;     // scale * log2(e): scores are kept in log2 units
    int splits;
    int by_stride;        // 1: runs of ceil(stride/splits) cache rows; 0: ceil(len/splits)
    int q4;               // 1: the cache is q4_0 (18-byte blocks), 0: q8_0
    int legacy_body = 0;  // q8_0 value side: 0 the process-wide default, 1 mma.sync (selector 7),
                          // 2 tcgen05 kind::i8 (selector 8)
    int run_cap;          // tensor-core body, by_stride == 0: at most this many live runs per
                          // KV head, balanced to within one 64-key tile (0: the reference's runs)
    int share_slots;      // tensor-core body, several slots: the device's CTA slots, shared by
                          // all slots in proportion to their live lengths (0: off)
    int n_slots;          // set by launch_decode_tc
    // Optional fused append (tensor-core body, q8_0): the new K/V rows of every slot, f32
    // [n_kv][256] at k_row + slot * row_slot. The CTA whose run holds the append position
    // (the int before the live length in `len`) quantises the row into its tile and stores
    // it to the cache through kw / vw (the same addresses as k / v).
    const float *k_row = nullptr, *v_row = nullptr;
    unsigned char *kw = nullptr, *vw = nullptr;
    long long row_slot = 0;
    long long kv_slot_bytes, acc_slot, ml_slot, q_slot;
    // Fold inside the split pass (tensor-core body). The CTA that completes a group of eight
    // runs of a (slot, KV head) folds them into the group's first slot, and the CTA that
    // completes the last group folds the groups and writes the output rows of the head group,
    // so a decode step of a layer is one launch (a head with at most 30 runs is one group). The arrival counters live in library-owned
    // device memory (region `arrive_region`, `arrive_stride` counters per (slot, KV head):
    // one for the groups, then one per group) and return to zero by themselves.
    float *out = nullptr;            // nullptr: partials only, the caller launches the fold
    long long out_slot = 0, out_head_stride = 0;
    int normalize = 1;               // 0: out row = [acc (unnormalised) | max | sum]
    const float *gate = nullptr;     // optional, normalize only: out *= sigmoid(gate)
    int arrive_region = -1, arrive_stride = 0;
    // Sequence-split decode across GPUs: instead of writing `out` directly the folding CTA
    // stores the head group's (acc, max, sum) triples into every rank's table (phase bit 0),
    // and/or waits for all ranks' triples and folds them into `out` (phase bit 1).
    // by_head: head h's triples go only to rank h / (n_heads / shards), and only that rank
    // folds them and writes head h's output row (the layout a row-parallel output projection
    // wants); a rank's other output rows are left alone.
    struct Exchange {
        unsigned char *ws[16];
        int shards = 0, rank = 0, phases = 0;
        unsigned wait_us = 0;
        int by_head = 0;
    } xch;
};
// Live runs of one slot in the tensor-core split pass, in 64-key tiles: `runs` runs deal the
// slot's `tiles` tiles out to within one tile (run i covers tiles [i*tiles/runs,
// (i+1)*tiles/runs)). Single stream: min(splits, tiles, run_cap). Several slots sharing the
// device (share_slots > 0): every run gets `quota` tiles, about total_tiles * n_kv /
// share_slots, so a slot's runs are proportional to its live length and the whole batch is
// one round of CTAs; every slot has at least one run (a slot without rows gets one CTA per KV
// head, which writes the zero rows of its output). runs == -1: the reference's fixed runs
// apply instead.
struct RunPlan {
    int tiles, runs;
};
__host__ __device__ __forceinline__ int shared_runs_of(int tiles, int quota) {
    const int r = (tiles + quota - 1) / quota;
    return r < 1 ? 1 : r;
}
// Tiles per run of the shared plan: the smallest quota, not below ceil(longest / splits) (a
// head has `splits` partial slots), whose runs fit the share_slots CTAs that are launched.
// runs_at(q) returns the batch's run count per KV head at quota q (non-increasing in q);
// total / longest are the batch's tile sum and longest slot. The answer always fits:
// sum(max(1, ceil(t / q))) <= total / q + slots, so q = ceil(total / (fit - slots)) does, and
// the launchers take this plan only when 2 * slots * n_kv <= share_slots.
// (runs_at is a host lambda on the host and a device lambda on the device)
#pragma nv_exec_check_disable
template <class RunsAt>
__host__ __device__ __forceinline__ int solve_quota(int total, int longest, int slots, int splits,
                                                    int share_slots, int n_kv, RunsAt runs_at) {
    const int fit = share_slots / n_kv;   // runs per KV head that one round of CTAs holds
    int lo = (total + fit - 1) / fit;
    const int floor_q = (longest + splits - 1) / splits;
    if (lo < floor_q) lo = floor_q;
    if (lo < 1) lo = 1;
    if (runs_at(lo) <= fit) return lo;
    int hi = fit > slots ? (total + (fit - slots) - 1) / (fit - slots) : longest;
    if (hi < lo + 1) hi = lo + 1;
    // invariant: lo does not fit, hi does
    while (hi - lo > 1) {
        const int mid = lo + (hi - lo) / 2;
        if (runs_at(mid) <= fit) hi = mid; else lo = mid;
    }
    return hi;
}
#ifdef __CUDACC__
// Called by all 32 lanes of one warp (lane-strided over the slots); every lane returns the
// same value.
__device__ __forceinline__ int shared_quota_warp(const int *len, int len_stride, int len_offset,
                                                 int slots, int splits, int share_slots, int n_kv) {
    const int lane = threadIdx.x & 31;
    int total = 0, longest = 0;
    for (int s = lane; s < slots; s += 32) {
        const int t = (len[s * len_stride + len_offset] + 63) >> 6;
        total += t;
        longest = max(longest, t);
    }
    total = __reduce_add_sync(0xffffffffu, total);
    longest = __reduce_max_sync(0xffffffffu, longest);
    auto runs_at = [&](int q) {
        int runs = 0;
        for (int s = lane; s < slots; s += 32)
            runs += shared_runs_of((len[s * len_stride + len_offset] + 63) >> 6, q);
        return (int)__reduce_add_sync(0xffffffffu, runs);
    };
    return solve_quota(total, longest, slots, splits, share_slots, n_kv, runs_at);
}
// `quota`: shared_quota_warp's value when share_slots > 0 (unused otherwise).
__device__ __forceinline__ RunPlan plan_runs(const int *len, int len_stride, int len_offset, int slot,
                                             int splits, int run_cap, int share_slots, int quota) {
    RunPlan r;
    r.tiles = (len[slot * len_stride + len_offset] + 63) >> 6;
    if (share_slots > 0)
        r.runs = shared_runs_of(r.tiles, quota);
    else if (run_cap > 0)
        r.runs = min(min(splits, r.tiles), run_cap);
    else
        r.runs = -1;
    return r;
}
#endif
// The same quota from host-side lengths (the C ABI's hipml_decode_plan_quota).
int decode_plan_quota_host(const int *lens, int slots, int splits, int share_slots, int n_kv);

// Launches the split pass (the caller launches the reduce).
int launch_decode_split(cudaStream_t stream, const DecodeParams &p, int slots, bool tensor_core);
int launch_decode_tc(cudaStream_t stream, const DecodeParams &p, int slots);
// The fold of the tensor-core split pass as a launch of its own (the same arithmetic, bit for
// bit, as the fold inside the split pass): p.out and the fields after it say where it goes.
int launch_decode_fold_tree(cudaStream_t stream, const DecodeParams &p, int slots);
// Arrival-counter region for a launch on `stream` (-1: none free, use the two-launch form);
// `counters` = slots * n_kv * arrive_stride must fit a region.
int decode_arrive_region(cudaStream_t stream, long long counters);
constexpr int kFoldGroup = 8;          // runs per first-level group of the fold
constexpr int kFoldFlat = 30;          // up to this many runs a head is folded in one level
// Runs per first-level group for a head with `runs` live runs: few runs are one group (one
// arrival and up to three rounds of loads instead of two dependent levels).
__host__ __device__ __forceinline__ int fold_group_of(int runs) {
    return runs <= kFoldFlat ? 32 : kFoldGroup;
}
constexpr int kArriveRegionInts = 4096;
// Fold of (acc, max, sum) triples over the split axis; all strides in floats.
struct FoldParams {
    const float *acc;
    const float *ml;   // (max in log2 units, sum) pairs
    float *out;
    int head_dim, splits;
    long long acc_head_stride, acc_split_stride, ml_head_stride, ml_split_stride;
    long long acc_slot, ml_slot, out_slot, out_head_stride;
    int normalize;     // 1: out = acc/sum; 0: out row = [acc (unnormalised) | max | sum]
    const float *gate; // optional, normalize only: out *= sigmoid(gate), laid out as out
};
int launch_decode_fold(cudaStream_t stream, const FoldParams &p, int n_heads, int slots);
// Folds the partials into out[slot][h][d] (slot strides in floats).
int launch_decode_reduce(cudaStream_t stream, const float *part_acc, const float *part_ml,
                         float *out, int n_heads, int head_dim, int splits, int slots,
                         long long acc_slot, long long ml_slot, long long out_slot,
                         const float *gate = nullptr);

// Scalar chunk attention (attn_chunk_scalar.cu).
struct ChunkScalarParams {
    const float *q;
    const void *k;
    const void *v;
    float *out;        // splits < 2
    float *part_acc;   // splits >= 2
    float *part_ml;
    int n_heads, n_kv, head_dim;
    int pos0, tokens;
    int kv_dtype;      // 0 f32 position-major, 1 q8_0 head-major
    int stride;
    float scale_log2;
    int splits, qslots;
};
int launch_chunk_scalar(cudaStream_t stream, const ChunkScalarParams &p);
int launch_chunk_combine(cudaStream_t stream, const float *part_acc, const float *part_ml,
                         float *out, int n_heads, int head_dim, int tokens, int qslots, int splits,
                         const float *gate = nullptr);

// Throughput form of the q8_0 bulk append, head_dim 256 and 16-byte-aligned sources (kv_encode.cu).
int launch_kv_encode_bulk_rows(cudaStream_t stream, const float *k, const float *v,
                               unsigned char *kc, unsigned char *vc, int n_kv, int stride,
                               int start, int src0, int rows);

int launch_kv_encode_bulk_rows_q4(cudaStream_t stream, const float *k, const float *v,
                                  unsigned char *kc, unsigned char *vc, int n_kv, int stride,
                                  int start, int src0, int rows);

// Tensor-core chunk attention (attn_chunk_tc.cu).
size_t chunk_tc_workspace_bytes(int n_kv, int n_keys);
int launch_chunk_stage(cudaStream_t stream, const void *k_cache, const void *v_cache, int n_kv,
                       int kv_dtype, int stride, int key_from, int key_to, int cap,
                       void *workspace);
int launch_chunk_tc(cudaStream_t stream, const float *q, float *out, float *part_acc,
                    float *part_ml, int n_heads, int n_kv, int pos0, int tokens, int cap,
                    int splits, int variant, void *workspace, int *status,
                    const float *gate = nullptr);

// Sequence-split decode across GPUs (decode_exchange.cu): workspace size, and the collect
// half as a launch of its own (p.xch, p.out, p.n_heads are read).
size_t decode_exchange_bytes(int n_heads, int head_dim, int shards);
int launch_decode_collect(cudaStream_t stream, const DecodeParams &p, int *status);
// With more ranks than this the exchange is a launch of its own over (head, rank) CTAs.
constexpr int kInKernelShards = 2;
float *decode_exchange_stage(void *ws, int n_heads, int shards);
int launch_decode_exchange_wide(cudaStream_t stream, const DecodeParams &p, int *status);
void decode_set_two_launch_fold(int on);
void decode_set_body(int body);

// Attention front end and tail (attn_front.cu).
int launch_q_gate(cudaStream_t stream, const float *q, const float *gate, float *y, long long n);
int launch_front_rows_q8(cudaStream_t stream, const float *qg, const float *k, const float *v,
                         float *q, float *gate, float *k_out, const float *q_norm,
                         const float *k_norm, void *k_cache, void *v_cache, int n_heads, int n_kv,
                         int n_rot, const int *sections, const int *pos4, const int *step, int pos0,
                         int tokens, int stride, float theta_base, float eps);

// f32-cache decode for `rows` consecutive columns (attn_decode_f32.cu): split pass + fold.
int launch_decode_cols_f32(cudaStream_t stream, const float *q, const float *k, const float *v,
                           float *part_acc, float *part_ml, float *out, int n_heads, int n_kv,
                           int head_dim, int n_ctx, int pos0, int rows, int splits);

}  // namespace hipml
