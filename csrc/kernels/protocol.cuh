// Shared-memory ABI of the peer transport: limits, error codes, the symmetric segment layout,
// per-rank constants, kernel argument blocks, bounded waits and the intra-rank grid barrier
// (parity: the reference's mapped-host-memory ABI, csrc/kernels/host_staged/common.cuh:61-158 and
// advanced_common.cuh:15-129).
//
// All shared state lives in one *symmetric segment* per rank: the same layout
// at the same offsets on every rank, reachable from every peer through `RankConst::seg[]`.
// The segment is HBM mapped over NVLink for transport "peer" and registered host memory for
// transport "host_staged"; the kernels do not care which.
//
// Direction of every cross-rank access (all are stores into the *consumer's* segment, all
// polling is on local memory):
//   counts message, counts_flag   source -> destination
//   staged row, ready flag        source -> destination
//   ack (ring mode only)          destination -> source
//   done / cdone (reuse guard)    destination -> source
//   abort                         any rank -> every rank
//   combine row, cready flag      expert rank -> source rank
#pragma once

#include <cstddef>
#include <cstdint>

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#ifdef __CUDACC__
#include "ptx.cuh"
#endif

namespace bep {

constexpr int kMaxRanks = 16;
constexpr int kMaxTopk = 32;
constexpr int kMaxExperts = 4096;
constexpr int kMaxChannels = 128;
constexpr int kMaxVirtualRanks = 8;
constexpr int kMaxAlignment = 256;
constexpr int kMaxWarps = 16;  // 1 control + send + receive warps per channel CTA
constexpr int kFlagStride = 32;  // bytes between small per-rank flags (one sector each)
constexpr int kMaxSendStages = 4;   // shared-memory row buffers per send warp
constexpr int kMaxRowBuffers = 40;  // send warps x stages + receive warps of one channel CTA
constexpr int kRoleFieldCount = 16; // counters per warp in a profiling build

// Channels per group of the layout phase's two-level prefix, and the size of its scratch.
constexpr int kHistGroup = 16;
__host__ __device__ inline std::size_t hist_scratch_ints(int channels, int bins) {
    const std::size_t groups = static_cast<std::size_t>((channels + kHistGroup - 1) / kHistGroup);
    return static_cast<std::size_t>(channels) * bins + 2 * (groups + 1) * bins + 1;
}

// Row buffers a dispatch CTA needs: with dedicated sender CTAs a CTA is either all send warps or control + receive
// warps; without them every channel CTA holds both kinds.
__host__ __device__ inline int dispatch_row_buffer_count(int tx_warps, int rx_warps, int stages, int send_ctas) {
    const int send = tx_warps * stages;
    return send_ctas > 0 ? (send > rx_warps ? send : rx_warps) : send + rx_warps;
}
inline int dispatch_cta_warps(int tx_warps, int rx_warps, int send_ctas) {
    return send_ctas > 0 ? (tx_warps > 1 + rx_warps ? tx_warps : 1 + rx_warps) : 1 + tx_warps + rx_warps;
}

// Error codes (2, 11, 12, 15, 16, 18, 19 and 20 keep the numbers DeepEP-style callers already know).
enum ErrorCode : int {
    kOk = 0,
    kErrInvalidRouting = 2,    // context = token, detail = slot
    kErrReuseGuardWait = 11,   // a peer never finished the previous epoch (context = peer)
    kErrCountsWait = 12,       // a peer's counts message never arrived (context = peer)
    kErrRowWait = 15,          // a staged row / combine row never arrived (context = source)
    kErrCapacity = 16,         // expanded or unique capacity exceeded
    kErrSequence = 18,         // a row carries the wrong sequence
    kErrAlreadyAborted = 19,   // this rank failed in an earlier launch
    kErrEpochExhausted = 20,
    kErrGridBarrier = 21,      // CTAs of one rank did not meet
    kErrPeerAbort = 22,        // a peer published abort (context = peer)
    kErrCreditWait = 23,       // ring mode: slot never acknowledged (context = peer)
    kErrCopyEngine = 24,       // a bulk copy never completed
    kErrFusedSignalWait = 25,  // fused down-projection + combine: a peer's GEMM never signalled (context = peer)
    kErrFusedGemm = 26,        // fused down-projection + combine: this rank's GEMM gave up (detail = its status word)
    kErrInjectedAbort = 27,    // the abort-after test hook fired on this rank
};

enum StatField : int {
    kStatSourceTokens = 0,   // tokens written for at least one remote rank (source dedup, "U")
    kStatRemoteRows = 1,     // rows received from remote ranks (receiver dedup, "F")
    kStatDeliveries = 2,     // remote (token, rank) deliveries sent
    kStatEarlyRows = 3,      // rows pushed before this rank's receive prefix was ready
    kStatRxEmptyProbes = 4,  // receive probes that found nothing
    kStatCreditMisses = 5,   // ring mode: sends that had to wait for credit
    kStatLocalRows = 6,      // rows that stayed on this rank
    kStatRowsPublished = 7,  // ready flags written (local + remote)
};

__host__ __device__ inline std::size_t align_up(std::size_t v, std::size_t a) { return (v + a - 1) / a * a; }

__host__ __device__ inline std::uint64_t make_seq(std::uint64_t epoch, std::uint32_t index_plus_one) {
    return (epoch << 32) | index_plus_one;
}

// Per-row metadata that travels behind the payload.  16 + 12*K bytes, K = top-k.
//   int32 src_token; float scale; uint32 seq_epoch (low word of the dispatch epoch); uint32 seq_index (src_token + 1);
//   int32 expert[K] (global id or -1); int32 expert_ordinal[K]; float weight[K];
__host__ __device__ inline int meta_bytes_for(int topk) { return static_cast<int>(align_up(16 + 12 * topk, 16)); }

struct SegmentLayout {
    std::size_t size_bytes;
    // dispatch
    std::size_t done_off;         // u64 [P] stride kFlagStride : written by rank d, last epoch d fully consumed
    std::size_t abort_off;        // u64 [P] stride kFlagStride : written by rank s when it fails
    std::size_t counts_flag_off;  // u64 [P] stride kFlagStride : epoch of the counts message from s
    std::size_t counts_off;       // i32 [P][counts_stride]     : rank_counts[P] | expert_counts[El] | chan_counts[C]
    std::size_t ready_off;        // u64 [P][C][Q]
    std::size_t ack_off;          // u64 [P][C][Q] (ring mode; in the *source's* segment, written by dest d)
    std::size_t stage_off;        // bytes [P][C][Q][row_stride]
    // combine
    std::size_t cdone_off;        // u64 [P] stride kFlagStride
    std::size_t cready_off;       // u64 [P][Tmax]
    std::size_t cstage_off;       // bytes [P][Tmax][crow_stride]
    // fused down-projection + combine: the GEMM epilogue of the expert's rank writes weighted output rows
    // straight into the token owner's slots; the owner sums its K slots per token
    std::size_t csig_off;         // u64 [P] stride kFlagStride : combine with a separate reduction: rank r has pushed all its rows of this epoch
    std::size_t fsig_off;         // u64 [P] stride kFlagStride : written by rank r's GEMM, epoch whose rows are all here
    std::size_t fdone_off;        // u64 [P] stride kFlagStride : written by rank d's reduction, last epoch it has consumed
    std::size_t fstage_off;       // bytes [Tmax][K][crow_stride]
    // relay (host_staged + numa_mode relay): outbox rows are written here by the owner and
    // forwarded by CPU threads; unused otherwise
    std::size_t relay_off;
    int num_ranks, num_channels, num_experts, num_local_experts, num_topk, hidden, num_max_tokens;
    int slots;           // Q: rows per (source, channel) ring
    int slots_full;      // ceil(Tmax / C): rows a channel can ever need
    int counts_stride;   // ints per counts message
    int row_stride;      // bytes per staged row
    int meta_off;        // BF16 rows: offset of the metadata inside the row = align16(H*2)
    int meta_off_fp8;    // FP8 rows: offset of the metadata = align16(H)
    int meta_bytes;
    int crow_stride;     // bytes per combine row = align128(H*2)
    int has_combine;
    int has_fused;
};

inline SegmentLayout make_segment_layout(int P, int C, int E, int K, int H, int Tmax, int payload_slots,
                                         bool with_combine, bool with_fused = false) {
    SegmentLayout l{};
    l.num_ranks = P;
    l.num_channels = C;
    l.num_experts = E;
    l.num_local_experts = E / P;
    l.num_topk = K;
    l.hidden = H;
    l.num_max_tokens = Tmax;
    l.slots_full = (Tmax + C - 1) / C;
    l.slots = payload_slots > 0 && payload_slots < l.slots_full ? payload_slots : l.slots_full;
    l.counts_stride = static_cast<int>(align_up(P + l.num_local_experts + C, 4));
    l.meta_bytes = meta_bytes_for(K);
    l.meta_off = static_cast<int>(align_up(static_cast<std::size_t>(H) * 2, 16));
    l.meta_off_fp8 = static_cast<int>(align_up(static_cast<std::size_t>(H), 16));
    l.row_stride = static_cast<int>(align_up(l.meta_off + l.meta_bytes, 128));
    l.crow_stride = static_cast<int>(align_up(static_cast<std::size_t>(H) * 2, 128));
    l.has_combine = with_combine ? 1 : 0;
    l.has_fused = with_fused ? 1 : 0;
    std::size_t off = 0;
    auto take = [&off](std::size_t bytes) {
        std::size_t at = off;
        off = align_up(off + bytes, 256);
        return at;
    };
    l.done_off = take(static_cast<std::size_t>(P) * kFlagStride);
    l.abort_off = take(static_cast<std::size_t>(P) * kFlagStride);
    l.counts_flag_off = take(static_cast<std::size_t>(P) * kFlagStride);
    l.counts_off = take(static_cast<std::size_t>(P) * l.counts_stride * 4);
    l.ready_off = take(static_cast<std::size_t>(P) * C * l.slots * 8);
    l.ack_off = take(static_cast<std::size_t>(P) * C * l.slots * 8);
    l.cdone_off = take(static_cast<std::size_t>(P) * kFlagStride);
    l.cready_off = take(with_combine ? static_cast<std::size_t>(P) * Tmax * 8 : 0);
    l.stage_off = take(static_cast<std::size_t>(P) * C * l.slots * l.row_stride);
    l.cstage_off = take(with_combine ? static_cast<std::size_t>(P) * Tmax * l.crow_stride : 0);
    l.csig_off = take(static_cast<std::size_t>(P) * kFlagStride);
    l.fsig_off = take(static_cast<std::size_t>(P) * kFlagStride);
    l.fdone_off = take(static_cast<std::size_t>(P) * kFlagStride);
    l.fstage_off = take(with_fused ? static_cast<std::size_t>(Tmax) * K * l.crow_stride : 0);
    l.relay_off = off;
    l.size_bytes = align_up(off, 4096);
    return l;
}

// Everything about one (virtual) rank that does not change between launches.  Lives in device
// memory; kernels receive a pointer.
struct RankConst {
    SegmentLayout lay;
    std::uint8_t* seg[kMaxRanks];  // seg[r] = base of rank r's segment as addressed from this rank
    int rank;
    int ring_mode;     // slots < slots_full: credit/ack path active
    int wire_fp8;      // remote rows travel as E4M3 + FP32 scale
    int recv_fp8;      // received rows stay E4M3 (row scale in recv_scale); every row is quantised, local ones too
    int use_tma;       // rows move with cp.async.bulk through shared memory
    int vec_ok;        // hidden*2 is a multiple of 16: 16-byte accesses are legal on rows
    int tx_warps, rx_warps;
    int send_stages;   // shared-memory row buffers per send warp (bulk-copy engine): 2, 3 or 4
    int fence_flags;   // READY flags of the send warps: 0 batches of rows behind one system-scope fence; 1 one fence per row, executed
                       // by the lane that waited for the copies (host segments); 2 one fence per row in every lane that stores a flag
                       // (the conservative setting)
    int send_ctas;     // CTAs beyond the channel CTAs that do nothing but send (0: the send warps sit in every channel CTA)
    int unique_cap, expanded_cap;
    int slot_smem_bytes;  // shared-memory bytes of one row buffer (TMA path)
    std::uint64_t timeout_ns;
    // persistent local state
    std::uint64_t* epochs;      // [0] dispatch epoch, [1] combine epoch, [2] first-error latch time
    unsigned long long* grid_bar;   // [0] dispatch barrier arrivals, [1] combine (monotonic)
    unsigned long long* done_ctas;  // [0] dispatch CTAs finished, [1] combine (monotonic)
    int* block_hist;            // scratch of the layout phase: per-channel counts [C][E + P], then two copies of the
                                // per-group and grand sums [2][groups + 1][E + P] and their generation (see hist_scratch_ints)
    std::uint64_t* plan_flags;  // [C] epoch whose routing plan channel c has finished writing (read by the sender CTAs)
    int* sticky;                // [0] != 0 once this rank has failed; [1..] first error record
    std::int64_t* chan_stats;   // [2][C + send CTAs][10]: per-CTA counters + start/end time; dispatch, then combine
    // test hooks (written by the host between launches; all zero in production)
    std::uint64_t delay_meta_ns, delay_tx_ns, delay_rx_ns, delay_scatter_ns, delay_prefix_ns;
    int test_skip_done_to;      // -1, else: do not publish `done` to this peer (mailbox-timeout test)
    int test_withhold_counts;   // != 0: never publish the counts message (prefix-timeout test)
    int test_corrupt_sequence;  // != 0: this rank's send warps write a wrong sequence into their rows (sequence-check test)
    std::uint64_t test_abort_after_ns;  // != 0: the control warp of channel 0 publishes an abort this long after the launch started
};

// One dispatch of one (virtual) rank.
struct DispatchArgs {
    const RankConst* rc;
    const __nv_bfloat16* x;        // [T, H]
    const std::int64_t* topk_idx;  // [T, K]
    const float* topk_w;           // [T, K] or nullptr (weights = 1)
    int num_tokens;
    int do_expand;
    int alignment;
    int zero_padding;
    int cached;  // plan already holds this routing: skip the layout phase
    // routing plan (one slot of the plan pool)
    std::uint32_t* plan_mask;  // [Tmax] destination rank mask per token
    int* plan_slot;            // [Tmax][P] channel-relative row index at each destination (-1: not sent)
    int* plan_expert_ord;      // [Tmax][K] stable ordinal of the token among this rank's tokens of that expert
    int* plan_counts;          // [P + E + C*P] totals per rank bin, per expert, then per (channel, rank)
    // outputs (one result pool)
    __nv_bfloat16* recv_x;
    std::int64_t* recv_idx;
    float* recv_w;
    float* recv_scale;             // [cap] row scales when rows stay E4M3 at the receiver
    std::int64_t* source_meta;     // [cap][3]
    int* comb_map;                 // [P*C*slots_full][2 + 2K]: inverse map for combine
    int* recv_chan_counts;         // [P][C]
    std::int64_t* unique_count;    // [1]
    std::int64_t* expanded_count;  // [1]
    int* expert_counts;            // [El]
    int* expert_offsets;           // [El+1]
    int* expert_prefix;            // [El]
    int* source_offsets;           // [P+1]
    int* source_expert_prefix;     // [P][El]
    int* error;                    // [8]
    std::int64_t* stats;           // [8]
    std::int64_t* timestamps;      // [2] transport start / end (globaltimer ns)
    std::int64_t* prefix_tx_ts;    // [C+1][2]
    std::int64_t* profile;         // [C][16] per-channel phase timestamps (globaltimer ns), see ProfilePoint
    std::int64_t* role_profile;    // [C][kMaxWarps][16] per-warp role counters (profiling builds only), or nullptr
};

// Phase timestamps every channel CTA leaves behind (one store each; always on).
enum ProfilePoint : int {
    kProfStart = 0,
    kProfGuardDone = 1,     // reuse guard satisfied (warp 0)
    kProfHistDone = 2,      // per-channel histogram written
    kProfBarrierDone = 3,   // grid barrier passed
    kProfPrefixScan = 4,    // exclusive prefix over channels done
    kProfCountsSent = 5,    // counts messages released (warp 1)
    kProfOrdinalsDone = 6,  // stable ordinals written (warp 0)
    kProfRolesSplit = 7,
    kProfCountsArrived = 8, // all P counts flags seen (control warp)
    kProfPrefixReady = 9,
    kProfFirstTxDone = 10,  // first token of send warp 0 published
    kProfTxDone = 11,       // send warp 0 finished its tokens
    kProfFirstRxRow = 12,   // receive warp 0 got its first row
    kProfRxDone = 13,       // receive warp 0 finished its rows
    kProfEnd = 14,
};

struct DispatchLaunch {
    int num_virtual;
    DispatchArgs r[kMaxVirtualRanks];
};

// One combine of one (virtual) rank: the inverse of a finished dispatch.
struct CombineArgs {
    const RankConst* rc;
    const __nv_bfloat16* y;       // expert outputs in the layout of the dispatch's recv_x
    const int* comb_map;          // from the dispatch result
    const int* recv_chan_counts;  // [P][C] from the dispatch result
    const std::uint32_t* plan_mask;  // [Tmax] of this rank's own tokens
    int num_tokens;               // this rank's own token count at dispatch
    int weighted;                 // apply dispatch-time weights (expanded layout)
    __nv_bfloat16* out;           // [T, H]
    int* error;                   // [8]
    std::int64_t* stats;          // [8]
    std::int64_t* profile;        // [C][8]: start, guard done, warp 0 expert side done, warp 0 source side done, end
};

struct CombineLaunch {
    int num_virtual;
    CombineArgs r[kMaxVirtualRanks];
};

// ---- ABI checks ----------------------------------------------------------------------------
// The host runtime (plain C++) fills these blocks and the kernels (nvcc) read them; a peer's kernels interpret
// this rank's segment with their own copy of SegmentLayout.  Pin sizes and key offsets so that a change on one
// side of either boundary cannot go unnoticed, and keep the by-value launch blocks inside the 4 KB kernel
// parameter space.
static_assert(sizeof(SegmentLayout) == 200 && offsetof(SegmentLayout, relay_off) == 120 &&
                  offsetof(SegmentLayout, num_ranks) == 128 && offsetof(SegmentLayout, has_fused) == 192,
              "SegmentLayout ABI changed");
static_assert(sizeof(RankConst) == 512 && offsetof(RankConst, seg) == 200 && offsetof(RankConst, rank) == 328 &&
                  offsetof(RankConst, timeout_ns) == 384 && offsetof(RankConst, epochs) == 392 &&
                  offsetof(RankConst, delay_meta_ns) == 448 && offsetof(RankConst, test_abort_after_ns) == 504,
              "RankConst ABI changed");
static_assert(sizeof(DispatchArgs) == 248 && offsetof(DispatchArgs, plan_mask) == 56 &&
                  offsetof(DispatchArgs, recv_x) == 88 && offsetof(DispatchArgs, role_profile) == 240,
              "DispatchArgs ABI changed");
static_assert(sizeof(CombineArgs) == 80, "CombineArgs ABI changed");
static_assert(sizeof(DispatchLaunch) <= 4096 && sizeof(CombineLaunch) <= 4096, "launch blocks must fit the kernel parameter space");
static_assert(16 + 12 * kMaxTopk <= 400, "row metadata of the largest top-k must fit its shared-memory staging area");
static_assert(kMaxRanks <= 32, "one lane per rank");
static_assert(kMaxTopk <= 32, "one lane per top-k slot");

#ifdef __CUDACC__

// ---- error recording -----------------------------------------------------------------------
// First error wins; later ones are dropped.  `sticky` survives the launch so that the next
// launch refuses to run (error 19), `error` belongs to the result pool of this launch.
__device__ __forceinline__ void record_error(const RankConst* rc, int* error, int code, int context, int detail) {
    if (atomicCAS(&error[0], 0, code) == 0) {
        error[1] = context;
        error[2] = detail;
        error[3] = static_cast<int>(blockIdx.x);
    }
    if (atomicCAS(&rc->sticky[0], 0, code) == 0) {
        rc->sticky[1] = context;
        rc->sticky[2] = detail;
        __threadfence();
        // tell every peer; all writers of abort[rank] belong to this rank and write the same fact
        for (int p = 0; p < rc->lay.num_ranks; ++p) {
            auto* flag = reinterpret_cast<std::uint64_t*>(rc->seg[p] + rc->lay.abort_off +
                                                          static_cast<std::size_t>(rc->rank) * kFlagStride);
            ptx::st_release_sys(flag, static_cast<std::uint64_t>(code));
        }
    }
}

// Bounded waiting.  One Health object per waiting warp/thread; `expired()` is called every few
// dozen polls and answers true when the caller must give up.  Order of checks: local failure
// latch (cheap), deadline, then every peer's abort flag (local memory, written remotely).
struct Health {
    const RankConst* rc;
    int* error;
    std::uint64_t deadline;
    unsigned polls;

    __device__ __forceinline__ Health(const RankConst* rc_, int* error_) : rc(rc_), error(error_), polls(0) {
        deadline = ptx::globaltimer_ns() + rc_->timeout_ns;
    }
    __device__ __forceinline__ bool failed() const { return ptx::ld_volatile(&rc->sticky[0]) != 0; }
    // returns true when the wait must end; records `code` on timeout
    __device__ bool expired(int code, int context, int detail) {
        if (failed()) return true;
        if (ptx::globaltimer_ns() > deadline) {
            record_error(rc, error, code, context, detail);
            return true;
        }
        for (int p = 0; p < rc->lay.num_ranks; ++p) {
            auto* flag = reinterpret_cast<const std::uint64_t*>(rc->seg[rc->rank] + rc->lay.abort_off +
                                                                static_cast<std::size_t>(p) * kFlagStride);
            if (p != rc->rank && ptx::ld_relaxed_sys(flag) != 0) {
                record_error(rc, error, kErrPeerAbort, p, static_cast<int>(ptx::ld_relaxed_sys(flag)));
                return true;
            }
        }
        return false;
    }
    // poll helper: call once per unsuccessful probe
    __device__ __forceinline__ bool give_up(int code, int context, int detail) {
        ++polls;
        if ((polls & 63u) == 0) {
            if (expired(code, context, detail)) return true;
        }
        if (polls > 16) ptx::nanosleep(polls > 1024 ? 256 : 32);
        return false;
    }
};

// Barrier over the CTAs of one rank (gridDim.x of them).  The arrival counter only grows and
// barriers of one rank never overlap (launches of one buffer are stream-ordered), so the
// arrival number itself tells which barrier this is: it completes at the next multiple of
// gridDim.x.  The launch is cooperative, so every CTA is resident; the spin is bounded by the
// protocol timeout.  Returns false when the rank has failed.
__device__ __forceinline__ bool grid_barrier(unsigned long long* counter, Health& health) {
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        const unsigned long long arrival = atomicAdd(counter, 1ull);
        const unsigned long long target = (arrival / gridDim.x + 1ull) * gridDim.x;
        while (*reinterpret_cast<volatile unsigned long long*>(counter) < target) {
            if (health.give_up(kErrGridBarrier, static_cast<int>(blockIdx.x), 0)) break;
        }
        __threadfence();
    }
    __syncthreads();
    return !health.failed();
}

__device__ __forceinline__ void test_delay(std::uint64_t ns) {
    if (ns == 0) return;
    const std::uint64_t until = ptx::globaltimer_ns() + ns;
    while (ptx::globaltimer_ns() < until) ptx::nanosleep(100);
}

__device__ __forceinline__ std::uint64_t* flag_ptr(std::uint8_t* seg, std::size_t off, int index) {
    return reinterpret_cast<std::uint64_t*>(seg + off + static_cast<std::size_t>(index) * kFlagStride);
}

#endif  // __CUDACC__

}  // namespace bep
