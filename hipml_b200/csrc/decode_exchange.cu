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
    const int e = *reinterpret_cast<volatile int *>(p.xch.ws[p.xch.rank]);
    const unsigned long long deadline = global_timer_ns() + 1000ull * p.xch.wait_us;
    FoldAcc f;
    if (exchange_collect_warp(p.xch, p.n_heads, h, e, deadline, lane, f))
        fold_emit(p, 0, h, f, lane, true);
    else if (lane == 0)
        atomicCAS(status, 0, 31);
}

}  // namespace

size_t decode_exchange_bytes(int n_heads, int head_dim, int shards) {
    return (size_t)kExchangeHeaderBytes + 2 * (size_t)shards * n_heads * (head_dim + 2) * 8;
}

int launch_decode_collect(cudaStream_t stream, const DecodeParams &p, int *status) {
    return launch_pdl(attn_decode_collect, dim3((p.n_heads + 7) / 8), dim3(256), 0, stream, 1, p, status);
}

}  // namespace hipml
