// The ordinary (non-cooperative, fully occupied) launches of the combine paths.
//
// combine_push_kernel -- expert side of `combine`: for every row this rank received in the dispatch, reduce the
//   expert outputs of that token with the dispatch-time weights in FP32, round to BF16 and store the partial row
//   straight into the token owner's landing area over NVLink (16-byte stores, 512 contiguous bytes per warp
//   instruction).  The launch's last CTA publishes the epoch to every owner.  Nothing in it waits on another
//   kernel of the same launch wave, so it needs no co-residency and any grid size works.  With one rank the
//   reduced rows are the result and go straight to `out`.
// fused_reduce_kernel -- owner side: producers on every rank have written weighted BF16 rows into this rank's
//   landing area and published their epoch; this kernel waits -- bounded -- for every rank's epoch, adds the rows
//   of every token in slot order (FP32, deterministic) and hands the area back.  Two producers use it:
//     * combine_push_kernel: one slot per (token, expert rank), valid where the token's destination mask has
//       that rank's bit;
//     * the fused down projection (expert_gemm.cu, scatter variant): one slot per (token, k), valid where the
//       routing plan's expert ordinal is >= 0.
#pragma once

#include "protocol.cuh"

namespace bep {

constexpr int kFusedReduceThreads = 256;

struct FusedReduceArgs {
    const RankConst* rc;
    const int* expert_ord;         // [Tmax][slots] routing plan of this rank's own tokens: -1 = unused slot; or nullptr
    const std::uint32_t* rank_mask;  // when expert_ord is null: [Tmax] destination mask, bit s = slot s is used
    const int* gemm_status;        // status word of this rank's own scatter GEMM of the same call (or nullptr)
    int num_tokens;
    std::uint64_t epoch;           // epoch every producer publishes (0: read the combine epoch rc->epochs[1])
    unsigned long long* cta_done;  // CTAs of this launch that have finished; the last one puts it back to zero
    std::size_t stage_off, sig_off, done_off;   // landing area, producers' flags, "consumed" flags (segment offsets)
    std::size_t slot_stride, token_stride;      // bytes between the slots of a token / between tokens
    int slots;                     // rows per token: top-k or number of ranks
    __nv_bfloat16* out;            // [T, H]
    int* error;                    // [8]
};

struct CombinePushArgs {
    const RankConst* rc;
    const __nv_bfloat16* y;        // expert outputs in the layout of the dispatch's recv_x
    const int* comb_map;           // [P][C][slots_full][2 + 2K]: token, n, then (row, weight bits) pairs
    const int* recv_chan_counts;   // [P][C] entries per (source, channel)
    const std::uint32_t* plan_mask;  // [Tmax] destination mask of this rank's own tokens (0: routed nowhere)
    int num_tokens;                // this rank's own token count at dispatch
    int weighted;
    __nv_bfloat16* out;            // [T, H]; written here only with a single rank
    int* error;                    // [8]
    std::int64_t* stats;           // [8]: rows pushed, of which to other ranks
    unsigned long long* cta_done;  // CTAs of this launch that have finished; the last one puts it back to zero
    unsigned long long* stat_scratch;  // [2] accumulators, zero between launches
};

#ifdef __CUDACC__

__device__ __forceinline__ void fused_accumulate(float (&acc)[8], const uint4& v) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(h[j]);
        acc[2 * j] += f.x;
        acc[2 * j + 1] += f.y;
    }
}

__global__ void __launch_bounds__(kFusedReduceThreads, 4) fused_reduce_kernel(const FusedReduceArgs a) {
    const RankConst* rc = a.rc;
    const SegmentLayout& lay = rc->lay;
    const int P = lay.num_ranks, K = a.slots;
    const std::uint64_t epoch = a.epoch != 0 ? a.epoch : rc->epochs[1];
    __shared__ int failed;
    if (threadIdx.x == 0) failed = 0;
    __syncthreads();
    if (static_cast<int>(threadIdx.x) < P) {
        const int peer = threadIdx.x;
        Health health(rc, a.error);
        const auto* flag = reinterpret_cast<const std::uint64_t*>(rc->seg[rc->rank] + a.sig_off +
                                                                  static_cast<std::size_t>(peer) * kFlagStride);
        while (ptx::ld_acquire_sys(flag) < epoch) {
            if (health.give_up(kErrFusedSignalWait, peer, 0)) {
                failed = 1;
                break;
            }
        }
    } else if (static_cast<int>(threadIdx.x) == P && a.gemm_status != nullptr) {
        const int status = ptx::ld_volatile(a.gemm_status);
        if (status != 0) {
            record_error(rc, a.error, kErrFusedGemm, rc->rank, status);
            failed = 1;
        }
    }
    __syncthreads();

    if (!failed) {
        // Work unit = (token, group of 32 sixteen-byte chunks): one warp iteration with up to 8 row loads per lane
        // in flight.  Units are dealt out in equal contiguous ranges so that every warp of the grid gets the same
        // share (a token per warp would leave the grid unbalanced at a few thousand tokens).
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        const int warps = kFusedReduceThreads / 32;
        const int chunks = lay.hidden * 2 / 16;
        const int groups = (chunks + 31) / 32;
        const long long units = static_cast<long long>(a.num_tokens) * groups;
        const long long total_warps = static_cast<long long>(gridDim.x) * warps;
        const long long me = static_cast<long long>(blockIdx.x) * warps + warp;
        const long long first = units * me / total_warps, last = units * (me + 1) / total_warps;
        const std::uint8_t* area = rc->seg[rc->rank] + a.stage_off;
        const std::size_t pitch = a.slot_stride;
        int cached_token = -1;
        unsigned valid = 0;
        for (long long u = first; u < last; ++u) {
            const int t = static_cast<int>(u / groups);
            const int c = static_cast<int>(u % groups) * 32 + lane;
            if (t != cached_token) {
                if (a.expert_ord != nullptr) {
                    const int ord = lane < K ? a.expert_ord[static_cast<std::size_t>(t) * K + lane] : -1;
                    valid = __ballot_sync(0xffffffffu, ord >= 0);
                } else {
                    valid = a.rank_mask[t];
                }
                cached_token = t;
            }
            if (c >= chunks) continue;
            const std::uint8_t* rows = area + static_cast<std::size_t>(t) * a.token_stride + static_cast<std::size_t>(c) * 16;
            float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            for (int k0 = 0; k0 < K; k0 += 8) {
                uint4 v[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int k = k0 + j;
                    v[j] = (k < K && (valid >> k & 1u)) ? ptx::ld_v4(rows + k * pitch) : make_uint4(0u, 0u, 0u, 0u);
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) fused_accumulate(acc, v[j]);
            }
            uint4 packed;
            __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
            for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
            reinterpret_cast<uint4*>(a.out + static_cast<std::size_t>(t) * lay.hidden)[c] = packed;
        }
    }

    // hand the landing area back: the launch's last CTA tells every rank that this epoch has been consumed
    __syncthreads();
    if (threadIdx.x == 0) {
        ptx::fence_sys();
        const unsigned long long finished = atomicAdd(a.cta_done, 1ull) + 1ull;
        if (finished == gridDim.x) {
            // launches that share this counter are stream-ordered: the next one finds it at zero again
            *a.cta_done = 0ull;
            ptx::fence_sys();
            for (int r = 0; r < P; ++r)
                ptx::st_release_sys(reinterpret_cast<std::uint64_t*>(rc->seg[r] + a.done_off +
                                                                     static_cast<std::size_t>(rc->rank) * kFlagStride),
                                    epoch);
        }
    }
}

// Work unit = (entry of the dispatch's combine map, group of 32 sixteen-byte chunks): one warp iteration with up to
// eight row loads per lane in flight.  Entries are numbered (channel, row index, source step) with the source
// fastest and rotated by this rank's index, so that at any moment a rank writes to all its peers at once and no
// owner is the target of every rank at the same time.  Units are dealt out in equal contiguous ranges.
__global__ void __launch_bounds__(kFusedReduceThreads, 3) combine_push_kernel(const CombinePushArgs a) {
    const RankConst* rc = a.rc;
    const SegmentLayout& lay = rc->lay;
    const int P = lay.num_ranks, C = lay.num_channels, Qf = lay.slots_full, K = lay.num_topk, H = lay.hidden;
    const int me = rc->rank;
    __shared__ int s_failed;
    __shared__ int s_max_rows;
    if (threadIdx.x == 0) {
        s_failed = 0;
        s_max_rows = 0;
    }
    __syncthreads();
    const bool aborted = ptx::ld_volatile(&rc->sticky[0]) != 0;
    const std::uint64_t epoch = rc->epochs[1] + 1;
    if (aborted) {
        if (threadIdx.x == 0) {
            if (blockIdx.x == 0) atomicCAS(&a.error[0], 0, kErrAlreadyAborted);
            s_failed = 1;
        }
    } else if (P > 1 && static_cast<int>(threadIdx.x) < P) {
        // reuse guard: an owner must have finished adding the previous combine's rows before new ones land
        Health health(rc, a.error);
        const std::uint64_t* done = flag_ptr(rc->seg[me], lay.cdone_off, threadIdx.x);
        while (ptx::ld_acquire_sys(done) + 1 < epoch) {
            if (health.give_up(kErrReuseGuardWait, threadIdx.x, 1)) {
                s_failed = 1;
                break;
            }
        }
    }
    // the longest (source, channel) list bounds the row index of the unit space
    {
        int local_max = 0;
        for (int i = threadIdx.x; i < P * C; i += blockDim.x) local_max = max(local_max, a.recv_chan_counts[i]);
        if (local_max > 0) atomicMax(&s_max_rows, local_max);
    }
    __syncthreads();

    unsigned long long pushed = 0, pushed_remote = 0;
    if (!s_failed) {
        const int map_stride = 2 + 2 * K;
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        const int warps = kFusedReduceThreads / 32;
        const int chunks = H * 2 / 16;
        const int groups = (chunks + 31) / 32;
        const int J = min(s_max_rows, Qf);
        const long long total_warps = static_cast<long long>(gridDim.x) * warps;
        const long long wid = static_cast<long long>(blockIdx.x) * warps + warp;
        const long long units = static_cast<long long>(C) * J * P * groups;
        const long long first = units * wid / total_warps, last = units * (wid + 1) / total_warps;
        const std::uint8_t* y = reinterpret_cast<const std::uint8_t*>(a.y);
        const std::size_t row_bytes = static_cast<std::size_t>(H) * 2;
        const std::size_t rank_stride = static_cast<std::size_t>(lay.num_max_tokens) * lay.crow_stride;
        long long cached_entry = -1;
        bool present = false;
        int n = 0, row_of_lane = 0;
        float weight_of_lane = 1.0f;
        std::uint8_t* dst_row = nullptr;
        for (long long u = first; u < last; ++u) {
            const long long entry = u / groups;  // = (c * J + j) * P + step
            if (entry != cached_entry) {
                cached_entry = entry;
                const int step = static_cast<int>(entry % P);
                const long long cj = entry / P;
                const int c = static_cast<int>(cj / J), j = static_cast<int>(cj % J);
                const int s = (me + 1 + step) % P;
                present = j < a.recv_chan_counts[s * C + c];
                if (present) {
                    const int* map = a.comb_map + ((static_cast<std::size_t>(s) * C + c) * Qf + j) * map_stride;
                    const int token = map[0];
                    n = map[1];
                    if (lane < n) {
                        row_of_lane = map[2 + 2 * lane];
                        weight_of_lane = a.weighted ? __int_as_float(map[3 + 2 * lane]) : 1.0f;
                    }
                    dst_row = P == 1 ? reinterpret_cast<std::uint8_t*>(a.out + static_cast<std::size_t>(token) * H)
                                     : rc->seg[s] + lay.cstage_off + static_cast<std::size_t>(me) * rank_stride +
                                           static_cast<std::size_t>(token) * lay.crow_stride;
                    // an entry spans `groups` units, possibly of two warps: it is counted with its first unit
                    if (lane == 0 && u % groups == 0) {
                        ++pushed;
                        if (s != me) ++pushed_remote;
                    }
                }
            }
            if (!present) continue;
            const int q = static_cast<int>(u % groups) * 32 + lane;
            float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            for (int k0 = 0; k0 < n; k0 += 8) {
                uint4 v[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int k = min(k0 + i, n - 1);
                    const int row = __shfl_sync(0xffffffffu, row_of_lane, k);
                    v[i] = (k0 + i < n && q < chunks) ? ptx::ld_nc_v4(y + static_cast<std::size_t>(row) * row_bytes + static_cast<std::size_t>(q) * 16)
                                                     : make_uint4(0u, 0u, 0u, 0u);
                }
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float w = __shfl_sync(0xffffffffu, weight_of_lane, min(k0 + i, n - 1));
                    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v[i]);
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float2 f = __bfloat1622float2(h[e]);
                        acc[2 * e] = fmaf(w, f.x, acc[2 * e]);
                        acc[2 * e + 1] = fmaf(w, f.y, acc[2 * e + 1]);
                    }
                }
            }
            if (q < chunks) {
                uint4 packed;
                __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
                for (int e = 0; e < 4; ++e) h[e] = __floats2bfloat162_rn(acc[2 * e], acc[2 * e + 1]);
                ptx::st_v4(dst_row + static_cast<std::size_t>(q) * 16, packed);
            }
        }
        if (P == 1) {
            // tokens that were routed nowhere have no map entry: their result is zero
            const long long zero_units = static_cast<long long>(a.num_tokens) * groups;
            for (long long u = zero_units * wid / total_warps; u < zero_units * (wid + 1) / total_warps; ++u) {
                const int t = static_cast<int>(u / groups);
                const int q = static_cast<int>(u % groups) * 32 + lane;
                if (a.plan_mask[t] == 0 && q < chunks)
                    reinterpret_cast<uint4*>(a.out + static_cast<std::size_t>(t) * H)[q] = make_uint4(0u, 0u, 0u, 0u);
            }
        }
        if (lane == 0 && pushed) {
            atomicAdd(&a.stat_scratch[0], pushed);
            atomicAdd(&a.stat_scratch[1], pushed_remote);
        }
    }

    // every thread's stores, then the CTA joins, then one thread fences at system scope and counts the CTA
    __syncthreads();
    if (threadIdx.x == 0) {
        ptx::fence_sys();
        const unsigned long long finished = atomicAdd(a.cta_done, 1ull) + 1ull;
        if (finished == gridDim.x) {
            *a.cta_done = 0ull;  // launches that share this counter are stream-ordered
            ptx::fence_sys();
            a.stats[0] = static_cast<std::int64_t>(a.stat_scratch[0]);
            a.stats[1] = static_cast<std::int64_t>(a.stat_scratch[1]);
            for (int i = 2; i < 8; ++i) a.stats[i] = 0;
            a.stat_scratch[0] = 0ull;
            a.stat_scratch[1] = 0ull;
            if (ptx::ld_volatile(&rc->sticky[0]) == 0) {
                if (P > 1)
                    for (int p = 0; p < P; ++p) ptx::st_release_sys(flag_ptr(rc->seg[p], lay.csig_off, me), epoch);
                rc->epochs[1] = epoch;
            }
        }
    }
}

#endif  // __CUDACC__

}  // namespace bep
