// Expert side of `combine`: an ordinary (non-cooperative) launch.
//
// combine_push_kernel: for every row this rank received in the dispatch, reduce the expert outputs of that token
//   with the dispatch-time weights in FP32, round to BF16 and deliver the partial row to the token owner's landing
//   area: reducer CTAs write it to a local outbox, a few forwarder CTAs of the same launch copy completed rows over
//   NVLink with bulk copies.  The launch's last CTA publishes the epoch to every owner (whose fused_reduce_kernel,
//   fused_reduce.cuh, then adds the ranks' rows).  With one rank the reduced rows are the result and go straight
//   to `out`.
#pragma once

#include "fused_reduce.cuh"

namespace bep {

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
    std::int64_t* stats;           // [8]: rows pushed, of which to other ranks, ns until the last reducer CTA / the last
                                   // forwarder CTA had finished (from the first CTA's start)
    unsigned long long* cta_done;  // CTAs of this launch that have finished; the last one puts it back to zero
    unsigned long long* stat_scratch;  // [5] accumulators (rows, remote rows, first start, last reducer end, last forwarder
                                       // end); zero between launches, the first start all ones
    // rows whose owner is another rank are reduced into a local outbox and forwarded by dedicated CTAs
    std::uint8_t* outbox;              // [P*C*slots_full][crow_stride], local memory
    unsigned long long* outbox_units;  // [P*C*slots_full] finished units of the row in the outbox; zero between launches
    int forward_ctas;                  // the first CTAs of the grid only forward; 0 with a single rank
    unsigned long long* next_unit;     // next entry to hand out to a reducer warp; zero between launches
    unsigned long long* forwarder_sms; // [kMaxSmTable] combine epoch in which SM i hosts a forwarder CTA
};

constexpr int kPushGroupsPerUnit = 4;
constexpr int kMaxSmTable = 256;
constexpr int kForwardWarps = 2;   // per forwarder CTA
constexpr int kForwardStages = 3;  // row buffers per forwarder warp: loads run two rows ahead of the row being sent

// dynamic shared memory of the push kernel: the forwarder warps' row buffers behind 128 bytes of mbarriers
__host__ __device__ inline std::size_t combine_push_tile_offset(const SegmentLayout& lay, int forward_ctas) {
    return forward_ctas > 0 ? 128 + static_cast<std::size_t>(kForwardWarps) * kForwardStages * lay.crow_stride : 0;
}
inline std::size_t combine_push_smem_bytes(const SegmentLayout& lay, int forward_ctas) {
    return combine_push_tile_offset(lay, forward_ctas);
}

#ifdef __CUDACC__

// Expert side of combine.  Work unit = (entry of the dispatch's combine map, four groups of 32 sixteen-byte
// chunks): one warp iteration keeps eight row loads per lane in flight, whether the entry reduces one expert row
// or eight.  Entries are numbered (channel, row index, source step) with the source fastest and rotated by this
// rank's index; reducer warps take entries one at a time from one counter, so the rows complete roughly in their
// numbering order.
//
// Where the reduced row goes:
//   * one rank: straight to `out`;
//   * owner = this rank: straight into this rank's own landing area (a local store);
//   * owner = another rank: into a local outbox row.  The first `forward_ctas` CTAs of the grid do nothing but
//     copy completed outbox rows to their owners (bulk load into shared memory, bulk store to the peer).  A few SMs
//     saturate NVLink, and an SM with remote stores in flight loses most of its load and store throughput, so
//     confining the remote stores to those CTAs lets every other SM reduce at full HBM speed.
// A forwarder learns that an outbox row is complete from a per-entry counter of finished units (bounded wait).
// Forwarders never hold up a reducer, and reducers never wait for anything but the reuse guard, so the launch
// needs no co-residency guarantee: it is an ordinary launch and any grid size works.
namespace push_detail {

struct Entry {
    bool present;
    int s, token, n, slot;  // owner rank, its token, expert rows to reduce, index of the entry in the combine map
};

// entry number -> (channel, row index, owner); `slot` addresses the combine map and the outbox
__device__ __forceinline__ Entry locate_entry(const CombinePushArgs& a, int P, int C, int Qf, long long entry, int J, int me) {
    Entry e;
    const int step = static_cast<int>(entry % P);
    const long long cj = entry / P;
    const int c = static_cast<int>(cj / J), j = static_cast<int>(cj % J);
    e.s = (me + 1 + step) % P;
    e.present = j < a.recv_chan_counts[e.s * C + c];
    e.slot = (e.s * C + c) * Qf + j;
    e.token = 0;
    e.n = 0;
    return e;
}

}  // namespace push_detail

__global__ void __launch_bounds__(kFusedReduceThreads, 2) combine_push_kernel(const CombinePushArgs a) {
    using namespace push_detail;
    const RankConst* rc = a.rc;
    const SegmentLayout& lay = rc->lay;
    const int P = lay.num_ranks, C = lay.num_channels, Qf = lay.slots_full, K = lay.num_topk, H = lay.hidden;
    const int me = rc->rank;
    const int F = a.forward_ctas;
    const bool forwarder = static_cast<int>(blockIdx.x) < F;
    extern __shared__ __align__(128) unsigned char push_smem[];
    __shared__ int s_failed;
    __shared__ int s_max_rows;
    // The segment table and the two layout values a row needs are copied out of global memory once: a load per row is
    // slow on a forwarder's SM (it queues behind that SM's stores to peers), and the compiler cannot keep values
    // read through `rc` in registers across the inline assembly of the copy loop.
    __shared__ std::uint8_t* s_seg[kMaxRanks];
    if (threadIdx.x == 0) {
        s_failed = 0;
        s_max_rows = 0;
    }
    if (threadIdx.x < kMaxRanks) s_seg[threadIdx.x] = static_cast<int>(threadIdx.x) < P ? rc->seg[threadIdx.x] : nullptr;
    const std::size_t crow_stride = lay.crow_stride, cstage_off = lay.cstage_off;
    __syncthreads();
    const bool aborted = ptx::ld_volatile(&rc->sticky[0]) != 0;
    const std::uint64_t epoch = rc->epochs[1] + 1;
    if (threadIdx.x == 0) atomicMin(&a.stat_scratch[2], ptx::globaltimer_ns());  // all ones between launches
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
    // the longest (source, channel) list bounds the row index of the entry space
    {
        int local_max = 0;
        for (int i = threadIdx.x; i < P * C; i += blockDim.x) local_max = max(local_max, a.recv_chan_counts[i]);
        if (local_max > 0) atomicMax(&s_max_rows, local_max);
    }
    __syncthreads();

    const int map_stride = 2 + 2 * K;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int warps = kFusedReduceThreads / 32;
    const int chunks = H * 2 / 16;
    const int groups = (chunks + 31) / 32;
    const int units_per_entry = (groups + kPushGroupsPerUnit - 1) / kPushGroupsPerUnit;
    const int J = min(s_max_rows, Qf);
    const long long entries = static_cast<long long>(C) * J * P;
    const std::size_t rank_stride = static_cast<std::size_t>(lay.num_max_tokens) * crow_stride;
    unsigned long long pushed = 0, pushed_remote = 0;

    if (!s_failed && forwarder) {
        // ---- forward completed outbox rows to their owners --------------------------------------------
        if (threadIdx.x == 0) {
            unsigned sm;
            asm volatile("mov.u32 %0, %%smid;" : "=r"(sm));
            if (sm < static_cast<unsigned>(kMaxSmTable)) ptx::st_relaxed_sys(reinterpret_cast<std::uint64_t*>(a.forwarder_sms + sm), epoch);
        }
        if (warp < kForwardWarps) {
            Health health(rc, a.error);
            const int fw = blockIdx.x * kForwardWarps + warp, fws = F * kForwardWarps;
            unsigned char* buffers = push_smem + 128 + static_cast<std::size_t>(warp) * kForwardStages * crow_stride;
            unsigned long long* bars = reinterpret_cast<unsigned long long*>(push_smem) + warp * kForwardStages;
            const bool issuer = lane == 31;
            const unsigned row_bytes = static_cast<unsigned>(H) * 2u;
            if (lane == 0)
                for (int i = 0; i < kForwardStages; ++i) ptx::mbar_init(reinterpret_cast<std::uint64_t*>(&bars[i]), 1);
            ptx::mbar_fence_init();
            __syncwarp();
            // Rows owned by other ranks, numbered like the entries but without the local owner's step; this warp
            // takes every fws-th of them, in increasing order (the order in which the reducers finish them).
            // Everything a row needs from global memory -- is the entry present, whose token is it, is the row
            // complete -- is fetched for 32 candidates at a time, one per lane: on an SM that is busy storing to
            // peers a dependent load per row would cost more than the row's copy.
            const long long remote_entries = static_cast<long long>(C) * J * (P - 1);
            long long batch_base = fw;   // remote-entry number of lane 0's candidate in the next batch
            unsigned todo = 0;           // lanes of the current batch whose rows still have to be forwarded
            int my_slot = 0, my_owner = 0, my_token = 0;
            bool my_ready = false;
            int issued = 0, sent = 0;
            std::uint8_t* dst_of[kForwardStages];
            bool ok = true;
            auto load_batch = [&]() {
                const long long q = batch_base + static_cast<long long>(lane) * fws;
                batch_base += 32ll * fws;
                bool present = false;
                my_ready = false;
                if (q < remote_entries) {
                    const int step = static_cast<int>(q % (P - 1));
                    const Entry e = locate_entry(a, P, C, Qf, (q / (P - 1)) * P + step, J, me);  // steps 0..P-2 are the other ranks
                    present = e.present;
                    if (present) {
                        my_slot = e.slot;
                        my_owner = e.s;
                        my_token = a.comb_map[static_cast<std::size_t>(e.slot) * map_stride];
                        my_ready = ptx::ld_acquire_gpu(reinterpret_cast<const std::uint64_t*>(a.outbox_units + e.slot)) >=
                                   static_cast<std::uint64_t>(units_per_entry);
                    }
                }
                todo = __ballot_sync(0xffffffffu, present);
            };
            // Start loading this warp's next row if there is one and it is complete.  `may_block`: wait (bounded) for
            // it to become complete; otherwise return at once when it is not, so that a loaded row is never held back.
            auto issue_next = [&](bool may_block) -> bool {
                while (todo == 0u) {
                    if (batch_base >= remote_entries) return false;
                    load_batch();
                }
                const int src = __ffs(todo) - 1;
                const int slot = __shfl_sync(0xffffffffu, my_slot, src);
                const int owner = __shfl_sync(0xffffffffu, my_owner, src);
                const int token = __shfl_sync(0xffffffffu, my_token, src);
                int state = __shfl_sync(0xffffffffu, my_ready ? 1 : 0, src);  // 1 complete, 0 not yet, -1 gave up
                if (state == 0) {
                    if (lane == 0) {
                        const auto* done_units = reinterpret_cast<const std::uint64_t*>(a.outbox_units + slot);
                        state = 1;
                        while (ptx::ld_acquire_gpu(done_units) < static_cast<std::uint64_t>(units_per_entry)) {
                            if (!may_block) {
                                state = 0;
                                break;
                            }
                            if (health.give_up(kErrRowWait, owner, slot)) {
                                state = -1;
                                break;
                            }
                        }
                    }
                    state = __shfl_sync(0xffffffffu, state, 0);
                    if (state == 1 && static_cast<int>(lane) == src) my_ready = true;
                }
                if (state < 0) ok = false;
                if (state != 1) return false;
                todo &= todo - 1;
                // every producer of this row has finished: its counter starts the next combine at zero
                if (lane == 0) a.outbox_units[slot] = 0ull;
                const int b = issued % kForwardStages;
                dst_of[b] = s_seg[owner] + cstage_off + static_cast<std::size_t>(me) * rank_stride +
                            static_cast<std::size_t>(token) * crow_stride;
                __syncwarp();  // the lane that saw the row complete, before the lane that copies it
                if (issuer) {
                    asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");  // the buffer's previous row has left it
                    ptx::mbar_expect_tx(reinterpret_cast<std::uint64_t*>(&bars[b]), row_bytes);
                    ptx::bulk_g2s(buffers + static_cast<std::size_t>(b) * crow_stride,
                                  a.outbox + static_cast<std::size_t>(slot) * crow_stride, row_bytes,
                                  reinterpret_cast<std::uint64_t*>(&bars[b]));
                }
                ++issued;
                return true;
            };
            while (ok) {
                // keep up to kForwardStages rows between "load issued" and "store issued"; only block for a row
                // when nothing is loaded
                while (ok && issued - sent < kForwardStages && issue_next(issued == sent)) {}
                if (!ok || issued == sent) break;
                const int b = sent % kForwardStages;
                while (!ptx::mbar_try_wait(reinterpret_cast<std::uint64_t*>(&bars[b]), static_cast<unsigned>(sent / kForwardStages) & 1u)) {
                    if (health.give_up(kErrCopyEngine, static_cast<int>(blockIdx.x), 1)) {
                        ok = false;
                        break;
                    }
                }
                ok = __all_sync(0xffffffffu, ok) != 0;
                if (!ok) break;
                if (issuer) {
                    ptx::bulk_s2g(dst_of[b], buffers + static_cast<std::size_t>(b) * crow_stride, row_bytes);
                    ptx::bulk_commit();
                }
                ++sent;
            }
            if (issuer) ptx::bulk_wait_all();  // every forwarded row has been performed at its owner
            // loads still in flight after a failure: give them a bounded time to land
            for (int r = sent; r < issued; ++r) {
                unsigned polls = 0;
                while (!ptx::mbar_try_wait(reinterpret_cast<std::uint64_t*>(&bars[r % kForwardStages]), static_cast<unsigned>(r / kForwardStages) & 1u) &&
                       ++polls < (1u << 20))
                    ptx::nanosleep(64);
            }
            if (!ok && lane == 0) s_failed = 1;
        }
    } else if (!s_failed) {
        // ---- reduce ----------------------------------------------------------------------------------------
        const long long total_warps = static_cast<long long>(gridDim.x - F) * warps;
        const long long wid = static_cast<long long>(blockIdx.x - F) * warps + warp;
        const std::uint8_t* y = reinterpret_cast<const std::uint8_t*>(a.y);
        const std::size_t row_bytes = static_cast<std::size_t>(H) * 2;
        // Entries are handed out one at a time through a counter (a warp reduces all units of its entry), so that rows
        // complete in roughly their numbering order -- the order in which the forwarders take them -- and so that
        // a slow reducer CTA is not left with a fixed share.  A reducer CTA that finds a forwarder on its own SM stops
        // taking entries: the two would hold each other up on the SM's one path to memory.
        // With fewer entries than warps (few tokens) an entry's units are shared out between several warps instead: a
        // row is then a handful of dependent round trips to memory for each of them, not one long chain for one warp.
        const int share = entries >= total_warps ? 1 : static_cast<int>(min(static_cast<long long>(units_per_entry), total_warps / max(entries, 1ll)));
        const int units_per_grab = (units_per_entry + share - 1) / share;
        const int parts = (units_per_entry + units_per_grab - 1) / units_per_grab;
        const unsigned long long grabs = static_cast<unsigned long long>(entries) * parts;
        unsigned long long* completed = nullptr;  // counter of the unit whose stores may still be in flight
        unsigned my_sm;
        asm volatile("mov.u32 %0, %%smid;" : "=r"(my_sm));
        int taken = 0, yields = 0;
        bool shares_sm = false;
        while (true) {
            if (F > 0 && !shares_sm && (taken++ & 3) == 0 && my_sm < static_cast<unsigned>(kMaxSmTable))
                shares_sm = ptx::ld_relaxed_sys(reinterpret_cast<const std::uint64_t*>(a.forwarder_sms + my_sm)) == epoch;
            if (shares_sm && yields < 128) {
                // stand aside (a few hundred microseconds at most, then help after all) and leave once every entry is taken
                ptx::nanosleep(2000);
                ++yields;
                if (ptx::ld_relaxed_sys(reinterpret_cast<const std::uint64_t*>(a.next_unit)) >= grabs) break;
                continue;
            }
            unsigned long long grabbed = 0;
            if (lane == 0) grabbed = atomicAdd(a.next_unit, 1ull);
            grabbed = __shfl_sync(0xffffffffu, grabbed, 0);
            if (grabbed >= grabs) break;
            const int part = static_cast<int>(grabbed % parts);
            Entry e = locate_entry(a, P, C, Qf, static_cast<long long>(grabbed / parts), J, me);
            if (!e.present) continue;
            const int* map = a.comb_map + static_cast<std::size_t>(e.slot) * map_stride;
            e.token = map[0];
            e.n = map[1];
            int row_of_lane = 0;
            float weight_of_lane = 1.0f;
            if (lane < e.n) {
                row_of_lane = map[2 + 2 * lane];
                weight_of_lane = a.weighted ? __int_as_float(map[3 + 2 * lane]) : 1.0f;
            }
            const bool remote = P > 1 && e.s != me;
            std::uint8_t* dst_row =
                P == 1 ? reinterpret_cast<std::uint8_t*>(a.out + static_cast<std::size_t>(e.token) * H)
                : remote ? a.outbox + static_cast<std::size_t>(e.slot) * crow_stride
                         : s_seg[me] + cstage_off + static_cast<std::size_t>(me) * rank_stride + static_cast<std::size_t>(e.token) * crow_stride;
            if (lane == 0 && part == 0) {
                ++pushed;
                if (remote) ++pushed_remote;
            }
            const int unit_end = min(units_per_entry, (part + 1) * units_per_grab);
            for (int unit = part * units_per_grab; unit < unit_end; ++unit) {
            const int q0 = unit * kPushGroupsPerUnit * 32 + lane;  // this lane's chunk in the unit's first group
            float acc[kPushGroupsPerUnit][8];
#pragma unroll
            for (int g = 0; g < kPushGroupsPerUnit; ++g)
#pragma unroll
                for (int x = 0; x < 8; ++x) acc[g][x] = 0.0f;
            // rows two at a time, four chunk groups each: eight 16-byte loads per lane in flight
            for (int i0 = 0; i0 < e.n; i0 += 2) {
                const int r0 = __shfl_sync(0xffffffffu, row_of_lane, i0);
                const int r1 = __shfl_sync(0xffffffffu, row_of_lane, min(i0 + 1, e.n - 1));
                const float w0 = __shfl_sync(0xffffffffu, weight_of_lane, i0);
                const float w1 = i0 + 1 < e.n ? __shfl_sync(0xffffffffu, weight_of_lane, min(i0 + 1, e.n - 1)) : 0.0f;
                const bool two = i0 + 1 < e.n;
                uint4 v0[kPushGroupsPerUnit], v1[kPushGroupsPerUnit];
#pragma unroll
                for (int g = 0; g < kPushGroupsPerUnit; ++g) {
                    const int q = q0 + g * 32;
                    v0[g] = q < chunks ? ptx::ld_nc_v4(y + static_cast<std::size_t>(r0) * row_bytes + static_cast<std::size_t>(q) * 16) : make_uint4(0u, 0u, 0u, 0u);
                    v1[g] = (two && q < chunks) ? ptx::ld_nc_v4(y + static_cast<std::size_t>(r1) * row_bytes + static_cast<std::size_t>(q) * 16) : make_uint4(0u, 0u, 0u, 0u);
                }
                if (completed != nullptr) {
                    // The previous unit's row went to the outbox: count it as finished now, while this unit's loads
                    // are on their way (its stores have had a whole unit's time to drain, so the fence is cheap).
                    if (lane == 0) {
                        __threadfence();
                        atomicAdd(completed, 1ull);
                    }
                    completed = nullptr;
                }
#pragma unroll
                for (int g = 0; g < kPushGroupsPerUnit; ++g) {
                    const __nv_bfloat162* h0 = reinterpret_cast<const __nv_bfloat162*>(&v0[g]);
                    const __nv_bfloat162* h1 = reinterpret_cast<const __nv_bfloat162*>(&v1[g]);
#pragma unroll
                    for (int x = 0; x < 4; ++x) {
                        const float2 f0 = __bfloat1622float2(h0[x]);
                        acc[g][2 * x] = fmaf(w0, f0.x, acc[g][2 * x]);
                        acc[g][2 * x + 1] = fmaf(w0, f0.y, acc[g][2 * x + 1]);
                    }
                    if (two) {
#pragma unroll
                        for (int x = 0; x < 4; ++x) {
                            const float2 f1 = __bfloat1622float2(h1[x]);
                            acc[g][2 * x] = fmaf(w1, f1.x, acc[g][2 * x]);
                            acc[g][2 * x + 1] = fmaf(w1, f1.y, acc[g][2 * x + 1]);
                        }
                    }
                }
            }
#pragma unroll
            for (int g = 0; g < kPushGroupsPerUnit; ++g) {
                const int q = q0 + g * 32;
                if (q < chunks) {
                    uint4 packed;
                    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
                    for (int x = 0; x < 4; ++x) h[x] = __floats2bfloat162_rn(acc[g][2 * x], acc[g][2 * x + 1]);
                    ptx::st_v4(dst_row + static_cast<std::size_t>(q) * 16, packed);
                }
            }
            if (remote) {
                // The row will be read by a bulk copy (asynchronous proxy) of a forwarder: every lane orders its ordinary
                // stores against that proxy here, on the writing side -- a proxy fence on a forwarder's SM would wait
                // behind that SM's stores to peers.  The warp joins; the unit is counted as finished one unit later.
                asm volatile("fence.proxy.async.global;" ::: "memory");
                __syncwarp();
                completed = a.outbox_units + e.slot;
            }
            }  // units of the entry
        }
        if (completed != nullptr && lane == 0) {
            __threadfence();
            atomicAdd(completed, 1ull);
        }
        if (P == 1) {
            // tokens that were routed nowhere have no map entry: their result is zero
            const long long zero_units = static_cast<long long>(a.num_tokens) * groups;
            for (long long u = wid; u < zero_units; u += total_warps) {
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
        atomicMax(&a.stat_scratch[forwarder ? 4 : 3], ptx::globaltimer_ns());
        ptx::fence_sys();
        const unsigned long long finished = atomicAdd(a.cta_done, 1ull) + 1ull;
        if (finished == gridDim.x) {
            *a.cta_done = 0ull;  // launches that share this counter are stream-ordered
            ptx::fence_sys();
            const unsigned long long first_start = a.stat_scratch[2];
            a.stats[0] = static_cast<std::int64_t>(a.stat_scratch[0]);
            a.stats[1] = static_cast<std::int64_t>(a.stat_scratch[1]);
            a.stats[2] = static_cast<std::int64_t>(a.stat_scratch[3] - first_start);
            a.stats[3] = a.stat_scratch[4] ? static_cast<std::int64_t>(a.stat_scratch[4] - first_start) : 0;
            for (int i = 4; i < 8; ++i) a.stats[i] = 0;
            for (int i = 0; i < 5; ++i) a.stat_scratch[i] = i == 2 ? ~0ull : 0ull;
            *a.next_unit = 0ull;
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
