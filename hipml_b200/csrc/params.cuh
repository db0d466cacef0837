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
};
// Live runs of one slot in the tensor-core split pass, in 64-key tiles: `runs` runs deal the
// slot's `tiles` tiles out to within one tile (run i covers tiles [i*tiles/runs,
// (i+1)*tiles/runs)). Single stream: min(splits, tiles, run_cap). Several slots sharing the
// device (share_slots > 0): every run gets `quota` tiles, about total_tiles * n_kv /
// share_slots, so a slot's runs are proportional to its live length and the whole batch is
// one round of CTAs. runs == -1: the reference's fixed runs apply instead.
struct RunPlan {
    int tiles, runs;
};
// Tiles per run of the shared plan. Called by all 32 lanes of one warp (lane-strided over
// the slots); every lane returns the same value.
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
    int quota = (total * n_kv + share_slots - 1) / share_slots;
    quota = max(max(quota, (longest + splits - 1) / splits), 1);
    // rounding every slot up can push the batch past one round of CTAs: grow the quota until
    // the live runs fit (a few steps; past `longest` every slot is one run)
    for (int step = 0; step < 64 && quota < longest; step++) {
        int runs = 0;
        for (int s = lane; s < slots; s += 32)
            runs += ((len[s * len_stride + len_offset] + 63) / 64 + quota - 1) / quota;
        runs = __reduce_add_sync(0xffffffffu, runs);
        if (runs * n_kv <= share_slots) break;
        quota++;
    }
    return quota;
}
// `quota`: shared_quota_warp's value when share_slots > 0 (unused otherwise).
__device__ __forceinline__ RunPlan plan_runs(const int *len, int len_stride, int len_offset, int slot,
                                             int splits, int run_cap, int share_slots, int quota) {
    RunPlan r;
    r.tiles = (len[slot * len_stride + len_offset] + 63) >> 6;
    if (share_slots > 0)
        r.runs = (r.tiles + quota - 1) / quota;
    else if (run_cap > 0)
        r.runs = min(min(splits, r.tiles), run_cap);
    else
        r.runs = -1;
    return r;
}

// Launches the split pass (the caller launches the reduce).
int launch_decode_split(cudaStream_t stream, const DecodeParams &p, int slots, bool tensor_core);
int launch_decode_tc(cudaStream_t stream, const DecodeParams &p, int slots);
int launch_decode_t5(cudaStream_t stream, const DecodeParams &p, int slots, int *status);
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
    // Optional: the partials come from the tensor-core split pass with balanced runs, which
    // leaves only min(splits, 64-key tiles of the live length, run_cap) live runs per head;
    // the rest are neutral and need not be read. len == nullptr: fold all `splits`.
    const int *len = nullptr;
    int len_stride = 0, len_offset = 0, run_cap = 0, share_slots = 0, n_kv = 1;
};
int launch_decode_fold(cudaStream_t stream, const FoldParams &p, int n_heads, int slots);
// Folds the partials into out[slot][h][d] (slot strides in floats).
int launch_decode_reduce(cudaStream_t stream, const float *part_acc, const float *part_ml,
                         float *out, int n_heads, int head_dim, int splits, int slots,
                         long long acc_slot, long long ml_slot, long long out_slot,
                         const float *gate = nullptr, const DecodeParams *live_runs = nullptr);

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

// Fold + peer-memory exchange + final fold of a sequence-split decode (decode_exchange.cu).
size_t decode_exchange_bytes(int n_heads, int head_dim, int shards);
int launch_decode_fold_exchange(cudaStream_t stream, const float *part_acc, const float *part_ml,
                                float *out, int n_heads, int head_dim, int splits,
                                void *const *peer_ws, int shards, int rank, int phases,
                                unsigned wait_limit_us, int *status,
                                const DecodeParams *live_runs = nullptr);

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
