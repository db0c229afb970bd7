// Fused expert-parallel dispatch: one cooperative launch per rank covers epoch bookkeeping, route
// validation, stable ordinals, the counts exchange, the all-to-all itself, receive-side expansion into
// per-expert rows, local-token handling, zero padding and statistics.
//
// Grid: (channels + send_ctas, virtual_ranks).  blockIdx.y picks the rank (more than one only when several
// ranks are emulated on one GPU).  blockIdx.x < channels is a channel CTA: channel c of a rank owns that rank's
// tokens [c*ceil(T/C), (c+1)*ceil(T/C)) and receives what channel c of every rank sent to it.  The CTAs beyond
// are dedicated senders: each pushes the remote rows of the channels c == its index (mod send_ctas).  With
// send_ctas == 0 the send warps sit inside every channel CTA instead.
//
// Warp roles inside a channel CTA:
//   warp 0              control: reuse guard, stable ordinals, receive prefix, zero padding
//   warps 1..tx         send: read a token row once, (quantise,) store it into the staging ring of
//                       every *remote* destination rank, then release that row's READY flag there.
//                       With the bulk-copy engine each send warp runs a software pipeline over a ring
//                       of `pipeline_stages` shared-memory row buffers: rows are loaded one or two
//                       tokens ahead, and READY flags are released at least two rows late, several rows
//                       at a time behind one system-scope fence, so neither the HBM read nor the NVLink
//                       round trip of one row holds up the next.
//   warps tx+1..        receive+expand: poll READY flags in local memory, read the staged row once
//                       and write it to every local expert row (or the unique row).  Rows whose
//                       destination is this rank itself never touch the staging ring: the receive
//                       warps take them straight from `x` whenever no remote row is waiting.
//
// Transport: a row crosses NVLink once per (token, destination rank) as posted stores into the
// destination's segment (16-byte stores, or cp.async.bulk from shared memory); every flag is
// written by exactly one rank and polled only by its owner in local memory.
//
// Files: dispatch_common.cuh (context, shared-memory layout, row helpers), dispatch_send.cuh (send roles),
// dispatch_receive.cuh (receive + expand role); this file holds the kernel itself: layout phases, control warp, epilogue.
#pragma once

#include "dispatch_common.cuh"
#include "dispatch_receive.cuh"
#include "dispatch_send.cuh"

namespace bep {

#ifdef __CUDACC__

// Two builds of the same kernel: CTAs of up to kSmallCtaThreads threads (every tuned configuration) get the larger
// register budget that one CTA per SM allows them, which keeps the receive role free of spills; wider CTAs take the
// other one.  The roles are instantiated per build so that each is compiled against its own kernel's budget.
constexpr int kSmallCtaThreads = 384;
template <int kCtaThreads>
__global__ void __launch_bounds__(kCtaThreads, 1) dispatch_kernel(const __grid_constant__ DispatchLaunch launch) {
    using namespace detail;
    const DispatchArgs& a = launch.r[blockIdx.y];
    const RankConst* __restrict__ rc = a.rc;
    const SegmentLayout& lay = rc->lay;

    const int P = lay.num_ranks, C = lay.num_channels, E = lay.num_experts, El = lay.num_local_experts;
    const int K = lay.num_topk, H = lay.hidden;
    const int me = rc->rank, c = blockIdx.x;
    const int S = rc->send_ctas;    // CTAs C .. C+S-1 of the grid only send (see send_role_bulk)
    const bool is_sender = c >= C;
    const int T = a.num_tokens;
    const int Tc = (T + C - 1) / C;
    const int t0 = is_sender ? 0 : min(T, c * Tc), t1 = is_sender ? 0 : min(T, t0 + Tc);
    const int warp = threadIdx.x >> 5;
    const unsigned lane = ptx::lane_id();
    const unsigned lt_mask = (1u << lane) - 1u;
    const unsigned full = 0xffffffffu;
    const int tx_warps = rc->tx_warps, rx_warps = rc->rx_warps;
    const bool vec_ok = rc->vec_ok != 0, use_tma = rc->use_tma != 0;
    const bool recv_fp8 = rc->recv_fp8 != 0;  // rows stay E4M3 at the receiver (scales in recv_scale); implies an FP8 wire
    const std::size_t out_row_bytes = static_cast<std::size_t>(H) * (recv_fp8 ? 1 : 2);
    std::uint8_t* const recv_bytes = reinterpret_cast<std::uint8_t*>(a.recv_x);

    extern __shared__ __align__(128) unsigned char smem_raw[];
    auto* sh = reinterpret_cast<DispatchShared*>(smem_raw);
    int* cnt_e = reinterpret_cast<int*>(smem_raw + align_up(sizeof(DispatchShared), 16));
    unsigned* bits_e = reinterpret_cast<unsigned*>(cnt_e + E);
    int* total_e = reinterpret_cast<int*>(bits_e + E);
    int* eoff = total_e + E;      // [El+1]
    int* ecount = eoff + El + 1;  // [El]
    int* spre = ecount + El;      // [P*El]
    const std::size_t msg_at = align_up(align_up(sizeof(DispatchShared), 16) + static_cast<std::size_t>(E) * 12 +
                                            static_cast<std::size_t>(El) * 8 + 4 + static_cast<std::size_t>(P) * El * 4,
                                        16);
    int* msg_sm = reinterpret_cast<int*>(smem_raw + msg_at);  // [P][counts_stride]: every source's counts message
    const std::size_t slots_at = align_up(msg_at + static_cast<std::size_t>(P) * lay.counts_stride * 4, 128);

    Health health(rc, a.error);
    const std::uint64_t epoch = rc->epochs[0] + 1;
    std::uint8_t* my_seg = rc->seg[me];
    std::int64_t* prof = a.profile + static_cast<std::size_t>(c) * 16;
#define BEP_PROF(point) prof[point] = static_cast<std::int64_t>(ptx::globaltimer_ns())
#if BEP_ENABLE_PROFILING
    // instrumented build: finer marks of the layout and prefix phases, in the (otherwise unused) counters of the control warp
    std::int64_t* const layout_marks = a.role_profile ? a.role_profile + static_cast<std::size_t>(c) * kMaxWarps * kRoleFields : nullptr;
#define BEP_LAYOUT_MARK(i) do { if (layout_marks) layout_marks[i] = static_cast<std::int64_t>(ptx::globaltimer_ns() - t_start); } while (0)
#else
#define BEP_LAYOUT_MARK(i) do {} while (0)
#endif

    // ---- launch-wide preconditions ---------------------------------------------------------------
    if (ptx::ld_volatile(&rc->sticky[0]) != 0) {
        // the whole rank takes this branch: the latch only changes while a launch is running
        if (threadIdx.x == 0 && c == 0) atomicCAS(&a.error[0], 0, kErrAlreadyAborted);
        return;
    }
    if (epoch >= (1ull << 32)) {
        if (threadIdx.x == 0) record_error(rc, a.error, kErrEpochExhausted, 0, 0);
        return;
    }
    if (threadIdx.x < 8) sh->stat[threadIdx.x] = 0;
    if (threadIdx.x == 0) {
        sh->prefix_ready = 0;
        sh->first_tx_ns = 0;
        sh->last_tx_ns = 0;
        ptx::mbar_init(reinterpret_cast<std::uint64_t*>(&sh->prefix_bar), 1);
        ptx::mbar_fence_init();
    }
    // one mbarrier per row buffer, each set up by a thread of its own (every path below joins the CTA before the roles split)
    if (use_tma && static_cast<int>(threadIdx.x) < dispatch_row_buffer_count(tx_warps, rx_warps, rc->send_stages, S)) {
        ptx::mbar_init(reinterpret_cast<std::uint64_t*>(&sh->mbar[threadIdx.x]), 1);
        ptx::mbar_fence_init();
    }
    // ---- the roles' context, in shared memory (the last thread writes it while the others start on the layout; every path joins the CTA before the roles split) ----------------
    Ctx& k = sh->ctx;
    if (threadIdx.x == blockDim.x - 1) {
        k.a = &a;
        k.rc = rc;
        k.sh = sh;
        k.eoff = eoff;
        k.spre = spre;
        k.row_buffers = smem_raw + slots_at;
        k.send_tiles = reinterpret_cast<int*>(smem_raw + slots_at + static_cast<std::size_t>(dispatch_row_buffer_count(tx_warps, rx_warps, rc->send_stages, S)) *
                                                                    static_cast<std::size_t>(align_up(lay.meta_off + lay.meta_bytes, 128)));
        k.my_seg = my_seg;
        k.recv_bytes = recv_bytes;
        k.prof = prof;
        k.role_prof = a.role_profile ? a.role_profile + static_cast<std::size_t>(c) * kMaxWarps * kRoleFields : nullptr;
        k.out_row_bytes = out_row_bytes;
        k.epoch = epoch;
        k.slot_bytes = static_cast<int>(align_up(lay.meta_off + lay.meta_bytes, 128));
        k.stages = rc->send_stages;
        k.P = P; k.C = C; k.E = E; k.El = El; k.K = K; k.H = H; k.Q = lay.slots; k.Qf = lay.slots_full;
        k.me = me; k.c = c; k.t0 = t0; k.t1 = t1; k.rx_warps = rx_warps;
        k.T = T; k.Tc = Tc;
        if (is_sender) {
            k.send_warps = tx_warps; k.send_first = c - C; k.send_stride = S;
        } else if (S == 0) {
            k.send_warps = tx_warps; k.send_first = c; k.send_stride = C;
        } else {
            k.send_warps = 0; k.send_first = C; k.send_stride = C;
        }
        k.rx_buffer_base = S == 0 ? tx_warps * rc->send_stages : 0;
        k.plan_is_foreign = is_sender;
        k.map_stride = 2 + 2 * K;
        k.vec_ok = vec_ok; k.use_tma = use_tma; k.wire_fp8 = rc->wire_fp8 != 0; k.recv_fp8 = recv_fp8;
        k.ring = rc->ring_mode != 0;
        k.fence_flags = rc->fence_flags != 0;
        k.fence_every_lane = rc->fence_flags == 2;
        k.corrupt_sequence = rc->test_corrupt_sequence != 0;
        k.expanded_cap = rc->expanded_cap;
        k.unique_cap = rc->unique_cap;
        k.delay_meta_ns = rc->delay_meta_ns;
        k.delay_tx_ns = rc->delay_tx_ns;
        k.delay_rx_ns = rc->delay_rx_ns;
        k.delay_scatter_ns = rc->delay_scatter_ns;
        k.timeout_ns = rc->timeout_ns;
        for (int p = 0; p < kMaxRanks; ++p) k.seg[p] = p < P ? rc->seg[p] : nullptr;
        k.lay = lay;
    }
    const unsigned long long t_start = ptx::globaltimer_ns();
    if (threadIdx.x == 0) {
        prof[kProfStart] = static_cast<std::int64_t>(t_start);
        prof[kProfFirstRxRow] = 0;
        prof[kProfFirstTxDone] = 0;
    }

    // Reuse guard: nothing of this epoch may reach a peer before that peer has finished reading the
    // previous epoch out of its segment.  The flags are local; the wait is normally free.
    if (warp == 0 && lane < static_cast<unsigned>(P)) {
        const std::uint64_t* done = flag_ptr(my_seg, lay.done_off, lane);
        while (ptx::ld_acquire_sys(done) + 1 < epoch) {
            if (health.give_up(kErrReuseGuardWait, lane, 0)) break;
        }
    }
    if (warp == 0) {
        __syncwarp();
        if (lane == 0) BEP_PROF(kProfGuardDone);
    }

    // ---- phase A: routing layout (skipped with a cached plan) ------------------------------------
    // O(T*K) work with one grid barrier: per-channel histograms, a prefix over channels, then ballots inside
    // 32-token chunks give every (token, bin) its stable ordinal.
    if (is_sender) {
        // a sender has no tokens of its own to lay out; it only takes part in the grid barrier
        if (!a.cached) grid_barrier(&rc->grid_bar[0], health);
    } else if (!a.cached) {
        // which copy of the running sums this layout uses (asked for now, needed after the histogram)
        const int generation = __ldcg(rc->block_hist + static_cast<std::size_t>(C) * (E + P) +
                                      static_cast<std::size_t>(2) * ((C + kHistGroup - 1) / kHistGroup + 1) * (E + P));
        for (int i = threadIdx.x; i < E; i += blockDim.x) {
            cnt_e[i] = 0;
            bits_e[i] = 0;
        }
        if (threadIdx.x < kMaxRanks) {
            sh->cnt_r[threadIdx.x] = 0;
            sh->bits_r[threadIdx.x] = 0;
        }
        __syncthreads();
        if (threadIdx.x == 0) BEP_LAYOUT_MARK(0);
        for (int t = t0 + threadIdx.x; t < t1; t += blockDim.x) {
            unsigned mask = 0;
            const std::int64_t* row = a.topk_idx + static_cast<std::size_t>(t) * K;
            for (int k0 = 0; k0 < K; k0 += 8) {
                std::int64_t e8[8];
                load_experts8(row + k0, K - k0, e8);
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const int k = k0 + u;
                    const std::int64_t e = e8[u];
                    if (k >= K || e == -1) continue;
                    bool bad = e < -1 || e >= E;
#pragma unroll
                    for (int u2 = 0; u2 < u; ++u2) bad = bad || e8[u2] == e;
                    for (int k2 = 0; k2 < k0 && !bad; ++k2) bad = row[k2] == e;
                    if (bad) {
                        record_error(rc, a.error, kErrInvalidRouting, t, k);
                        continue;
                    }
                    mask |= 1u << (static_cast<int>(e) / El);
                    atomicAdd(&cnt_e[e], 1);
                }
            }
            a.plan_mask[t] = mask;
            for (unsigned m = mask; m; m &= m - 1) atomicAdd(&sh->cnt_r[__ffs(m) - 1], 1);
        }
        if (threadIdx.x == 0) BEP_LAYOUT_MARK(1);
        __syncthreads();
        if (threadIdx.x == 0) BEP_LAYOUT_MARK(2);
        // Every CTA needs, per bin, the sum over the channels before it and the sum over all channels.  Reading all C
        // rows in every CTA makes the whole grid read the same lines at the same time, and those few L2 slices set
        // the pace.  So the counts are also added (fire-and-forget reductions) to a sum per group of kHistGroup channels
        // and to a grand total before the barrier; after it a CTA reads the grand total, the sums of the groups before
        // its own and the rows of the channels before it inside its group: 1 + C / kHistGroup + kHistGroup rows at most.
        const int W = E + P;
        const int groups = (C + kHistGroup - 1) / kHistGroup;
        int* const hist_rows = rc->block_hist;  // [C][W]
        int* const sums_base = rc->block_hist + static_cast<std::size_t>(C) * W;  // [2][groups + 1][W], then the generation
        // the sums are used alternately: this launch adds to one copy and clears the other for the next layout
        int* const sums = sums_base + static_cast<std::size_t>(generation & 1) * (groups + 1) * W;
        int* const sums_next = sums_base + static_cast<std::size_t>((generation + 1) & 1) * (groups + 1) * W;
        for (int i = threadIdx.x; i < W; i += blockDim.x) {
            const int v = i < E ? cnt_e[i] : sh->cnt_r[i - E];
            hist_rows[static_cast<std::size_t>(c) * W + i] = v;
            if (v != 0) {
                atomicAdd(sums + static_cast<std::size_t>(c / kHistGroup) * W + i, v);
                atomicAdd(sums + static_cast<std::size_t>(groups) * W + i, v);
            }
        }
        for (int i = c * static_cast<int>(blockDim.x) + threadIdx.x; i < (groups + 1) * W; i += C * static_cast<int>(blockDim.x)) sums_next[i] = 0;
        // Every thread makes its own reductions and stores visible to the GPU before it joins the barrier.  The
        // barrier's one fence (by thread 0, behind the CTA barrier) was enough while the scratch was written with plain
        // stores; with reductions in flight from the CTA's last warps it was not on every machine: on one four-GPU box
        // the bins of the highest experts -- the last warps' -- came out short and rows collided at the receiver.
        __threadfence();
        if (threadIdx.x == 0) BEP_PROF(kProfHistDone);
        grid_barrier(&rc->grid_bar[0], health);
        if (threadIdx.x == 0) BEP_PROF(kProfBarrierDone);
        // exclusive prefix over earlier channels (stable order = channel order = token order)
        for (int i = threadIdx.x; i < W; i += blockDim.x) {
            const int my_group = c / kHistGroup;
            int base = 0;
            const int total = __ldcg(sums + static_cast<std::size_t>(groups) * W + i);
            for (int g0 = 0; g0 < my_group; g0 += 8) {
                int v[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) v[u] = g0 + u < my_group ? __ldcg(sums + static_cast<std::size_t>(g0 + u) * W + i) : 0;
#pragma unroll
                for (int u = 0; u < 8; ++u) base += v[u];
            }
            {
                int v[kHistGroup];
#pragma unroll
                for (int u = 0; u < kHistGroup; ++u) {
                    const int c2 = my_group * kHistGroup + u;
                    v[u] = c2 < c ? __ldcg(hist_rows + static_cast<std::size_t>(c2) * W + i) : 0;
                }
#pragma unroll
                for (int u = 0; u < kHistGroup; ++u) base += v[u];
            }
            if (i < E) {
                cnt_e[i] = base;
                total_e[i] = total;
            } else {
                sh->cnt_r[i - E] = 0;  // row indices at a destination are channel-relative
                sh->total_r[i - E] = total;
            }
        }
        if (threadIdx.x == 0) BEP_LAYOUT_MARK(3);
        __syncthreads();
        if (threadIdx.x == 0) BEP_PROF(kProfPrefixScan);
        if (c == 0) {  // keep the totals with the plan so a cached dispatch can skip all of the above
            for (int i = threadIdx.x; i < P + E; i += blockDim.x)
                a.plan_counts[i] = i < P ? sh->total_r[i] : total_e[i - P];
            for (int i = threadIdx.x; i < C * P; i += blockDim.x)
                a.plan_counts[P + E + i] = __ldcg(rc->block_hist + static_cast<std::size_t>(i / P) * (E + P) + E + i % P);
        }
    } else {
        for (int i = threadIdx.x; i < P + E; i += blockDim.x) {
            if (i < P) sh->total_r[i] = a.plan_counts[i];
            else total_e[i - P] = a.plan_counts[i];
        }
        __syncthreads();
    }
    // Two things happen side by side before the roles split: warp 1 tells every destination what to
    // expect (counts message; channel d, d+C, ... serves destination d), warp 0 numbers this channel's tokens.
    if (warp == 1 && !is_sender && !rc->test_withhold_counts) {
        for (int d = c; d < P; d += C) {
            int* msg = reinterpret_cast<int*>(rc->seg[d] + lay.counts_off) + static_cast<std::size_t>(me) * lay.counts_stride;
            for (int i = lane; i < P + El + C; i += 32) {
                int v;
                if (i < P) v = sh->total_r[i];
                else if (i < P + El) v = total_e[d * El + (i - P)];
                else if (a.cached) v = a.plan_counts[P + E + (i - P - El) * P + d];
                else v = __ldcg(rc->block_hist + static_cast<std::size_t>(i - P - El) * (E + P) + E + d);
                msg[i] = v;
            }
            __syncwarp();
            if (lane == 0) ptx::st_release_sys(flag_ptr(rc->seg[d], lay.counts_flag_off, me), epoch);
        }
        if (lane == 0) BEP_PROF(kProfCountsSent);
    }
    if (!a.cached && !is_sender) {
    if (warp == 0) {
        // Stable ordinals, 32 tokens at a time: lane = token.  bits_*[bin] collects which lanes hit a
        // bin; an ordinal is (tokens before this chunk) + (lower lanes in the bin).
        for (int base_t = t0; base_t < t1; base_t += 32) {
            const int t = base_t + lane;
            const bool active = t < t1;
            const std::int64_t* row = a.topk_idx + static_cast<std::size_t>(active ? t : 0) * K;
            // The ids of the first eight choices are loaded once and stay in registers for all four passes; further
            // choices (top-k above 8) are read again in every pass.  The destination mask is rebuilt from the ids
            // (entries the histogram refused are refused here as well: a launch with such an entry has failed
            // already and its plan is never used).
            if (lane == 0) BEP_LAYOUT_MARK(4);
            std::int64_t first8[8];
            load_experts8(row, active ? K : 0, first8);
            auto ids_of_group = [&](int k0, std::int64_t (&e8)[8]) {
                if (k0 == 0) {
#pragma unroll
                    for (int u = 0; u < 8; ++u) e8[u] = first8[u];
                } else {
                    load_experts8(row + k0, active ? K - k0 : 0, e8);
                }
            };
            unsigned mask = 0;
            for (int k0 = 0; k0 < K; k0 += 8) {
                std::int64_t e8[8];
                ids_of_group(k0, e8);
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const std::int64_t e = e8[u];
                    if (e >= 0 && e < E) {
                        atomicOr(&bits_e[e], 1u << lane);
                        mask |= 1u << (static_cast<int>(e) / El);
                    }
                }
            }
            for (unsigned m = mask; m; m &= m - 1) atomicOr(&sh->bits_r[__ffs(m) - 1], 1u << lane);
            __syncwarp();
            if (lane == 0) BEP_LAYOUT_MARK(5);
            for (int k0 = 0; k0 < K; k0 += 8) {
                std::int64_t e8[8];
                ids_of_group(k0, e8);
                int ord8[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const std::int64_t e = e8[u];
                    ord8[u] = (e >= 0 && e < E) ? cnt_e[e] + __popc(bits_e[e] & lt_mask) : -1;
                }
                if (active) {
                    int* out = a.plan_expert_ord + static_cast<std::size_t>(t) * K + k0;
                    if (K - k0 >= 8 && (reinterpret_cast<std::uintptr_t>(out) & 15u) == 0) {
                        reinterpret_cast<int4*>(out)[0] = make_int4(ord8[0], ord8[1], ord8[2], ord8[3]);
                        reinterpret_cast<int4*>(out)[1] = make_int4(ord8[4], ord8[5], ord8[6], ord8[7]);
                    } else {
#pragma unroll
                        for (int u = 0; u < 8; ++u)
                            if (k0 + u < K) out[u] = ord8[u];
                    }
                }
            }
            if (active) {
                for (int d = 0; d < P; ++d)
                    a.plan_slot[static_cast<std::size_t>(t) * P + d] =
                        (mask >> d & 1u) ? sh->cnt_r[d] + __popc(sh->bits_r[d] & lt_mask) : -1;
            }
            __syncwarp();
            if (lane == 0) BEP_LAYOUT_MARK(6);
            for (int k0 = 0; k0 < K; k0 += 8) {
                std::int64_t e8[8];
                ids_of_group(k0, e8);
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const std::int64_t e = e8[u];
                    if (e >= 0 && e < E) {
                        const unsigned b = bits_e[e];
                        if (lane == 31u - __clz(b)) cnt_e[e] += __popc(b);
                    }
                }
            }
            for (unsigned m = mask; m; m &= m - 1) {
                const int d = __ffs(m) - 1;
                const unsigned b = sh->bits_r[d];
                if (lane == 31u - __clz(b)) sh->cnt_r[d] += __popc(b);
            }
            __syncwarp();
            if (lane == 0) BEP_LAYOUT_MARK(7);
            for (int k0 = 0; k0 < K; k0 += 8) {
                std::int64_t e8[8];
                ids_of_group(k0, e8);
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const std::int64_t e = e8[u];
                    if (e >= 0 && e < E) bits_e[e] = 0;
                }
            }
            for (unsigned m = mask; m; m &= m - 1) sh->bits_r[__ffs(m) - 1] = 0;
            __syncwarp();
        }
    }
        if (warp == 0 && lane == 0) {
            BEP_PROF(kProfOrdinalsDone);
            if (S > 0) {
                // this channel's plan is complete (the masks were written before the barrier above): the senders may read it
                __threadfence();
                ptx::st_release_gpu(&rc->plan_flags[c], epoch);
            }
        }
    }
    if (cta_failed(health, &sh->cta_flag)) return;
    if (threadIdx.x == 0) BEP_PROF(kProfRolesSplit);

    // ---- role split ------------------------------------------------------------------------------
    RoleStats st;

    if (is_sender) {
        // ===== dedicated sender: every warp sends =====
        if (warp < tx_warps) {
            if (!use_tma) send_role_vector<kCtaThreads>(k, warp, health, st);
            else if (k.stages >= 4) send_role_bulk<4, kCtaThreads>(k, warp, health, st);
            else if (k.stages == 3) send_role_bulk<3, kCtaThreads>(k, warp, health, st);
            else send_role_bulk<2, kCtaThreads>(k, warp, health, st);
            if (lane == 0) atomicMax(&sh->last_tx_ns, ptx::globaltimer_ns());
            if (warp == 0 && lane == 0) BEP_PROF(kProfTxDone);
        }
    } else if (warp == 0) {
        // ===== control: receive prefix from every source's counts message, then zero padding =====
        const unsigned long long prefix_t0 = ptx::globaltimer_ns();
        // test hook: this rank publishes an abort in mid-transfer (a legal owner writing its own abort flag) while
        // its send warps and its peers are busy
        if (c == 0 && rc->test_abort_after_ns != 0) {
            while (ptx::globaltimer_ns() < t_start + rc->test_abort_after_ns) ptx::nanosleep(200);
            if (lane == 0) record_error(rc, a.error, kErrInjectedAbort, me, 0);
            __syncwarp();
        }
        // what the prefix needs from the rank's constants is read while the counts are still on their way
        const int expanded_cap = rc->expanded_cap, unique_cap = rc->unique_cap;
        const std::uint64_t delay_prefix_ns = rc->delay_prefix_ns;
        bool gave_up = false;
        if (lane < static_cast<unsigned>(P)) {
            const std::uint64_t* flag = flag_ptr(my_seg, lay.counts_flag_off, lane);
            while (ptx::ld_acquire_sys(flag) != epoch) {
                if (health.give_up(kErrCountsWait, lane, 0)) {
                    gave_up = true;
                    break;
                }
            }
        }
        __syncwarp();
        if (lane == 0) BEP_PROF(kProfCountsArrived);
        test_delay(delay_prefix_ns);
        // (a wait that ended without its flag has latched the failure; the latch itself is looked at again below)
        const bool bad = __any_sync(full, gave_up) != 0;
        if (!bad) {
            const int stride = lay.counts_stride;
            {   // bring all P messages into shared memory with wide, independent loads
                const uint4* g = reinterpret_cast<const uint4*>(my_seg + lay.counts_off);
                uint4* d4 = reinterpret_cast<uint4*>(msg_sm);
                const int n4 = P * stride / 4;
                // eight loads per lane on their way before the first is stored: one round trip per 4 KB, not per 512 bytes
                for (int i0 = 0; i0 < n4; i0 += 256) {
                    uint4 v[8];
#pragma unroll
                    for (int u = 0; u < 8; ++u) {
                        const int i = i0 + u * 32 + static_cast<int>(lane);
                        v[u] = i < n4 ? ptx::ld_v4(g + i) : make_uint4(0u, 0u, 0u, 0u);
                    }
#pragma unroll
                    for (int u = 0; u < 8; ++u) {
                        const int i = i0 + u * 32 + static_cast<int>(lane);
                        if (i < n4) d4[i] = v[u];
                    }
                }
            }
            __syncwarp();
            if (lane == 0) BEP_LAYOUT_MARK(8);
            const int* msg = msg_sm;
            for (int el = lane; el < El; el += 32) {
                int run = 0;
                for (int s = 0; s < P; ++s) {
                    spre[s * El + el] = run;
                    run += msg[s * stride + P + el];
                }
                ecount[el] = run;
            }
            __syncwarp();
            // aligned exclusive scan over local experts, 32 at a time
            int carry = 0, true_total = 0;
            for (int e0 = 0; e0 < El; e0 += 32) {
                const int el = e0 + lane;
                const int cnt = el < El ? ecount[el] : 0;
                const int padded = (cnt + a.alignment - 1) / a.alignment * a.alignment;
                int incl = padded, tsum = cnt;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const int v = __shfl_up_sync(full, incl, o);
                    const int w = __shfl_up_sync(full, tsum, o);
                    if (lane >= static_cast<unsigned>(o)) {
                        incl += v;
                        tsum += w;
                    }
                }
                if (el < El) eoff[el] = carry + incl - padded;
                carry += __shfl_sync(full, incl, 31);
                true_total += __shfl_sync(full, tsum, 31);
            }
            if (lane == 0) eoff[El] = carry;
            if (lane == 0) BEP_LAYOUT_MARK(9);
            // unique layout: rows grouped by source rank
            const int from = lane < static_cast<unsigned>(P) ? msg[lane * stride + me] : 0;
            int incl = from;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int v = __shfl_up_sync(full, incl, o);
                if (lane >= static_cast<unsigned>(o)) incl += v;
            }
            if (lane < static_cast<unsigned>(P)) sh->source_offsets[lane] = incl - from;
            const int unique_total = __shfl_sync(full, incl, P - 1);
            if (lane == 0) sh->source_offsets[P] = unique_total;
            if (lane < static_cast<unsigned>(P)) {
                const int* chan = msg + lane * stride + P + El;
                int before = 0;
                for (int c2 = 0; c2 < c; ++c2) before += chan[c2];
                sh->chan_base[lane] = before;
                sh->chan_expected[lane] = chan[c];
                a.recv_chan_counts[lane * C + c] = sh->chan_expected[lane];
            }
            if (lane == 0) BEP_LAYOUT_MARK(10);
            if (carry > expanded_cap || unique_total > unique_cap) {
                if (lane == 0) record_error(rc, a.error, kErrCapacity, carry, unique_total);
            }
            __syncwarp();
            if (c == 0) {
                for (int el = lane; el < El; el += 32) {
                    a.expert_counts[el] = ecount[el];
                    a.expert_offsets[el] = eoff[el];
                    a.expert_prefix[el] = eoff[el] + ecount[el];
                }
                for (int i = lane; i < P * El; i += 32) a.source_expert_prefix[i] = spre[i];
                if (lane <= static_cast<unsigned>(P)) a.source_offsets[lane] = sh->source_offsets[lane];
                if (lane == 0) {
                    a.expert_offsets[El] = carry;
                    a.unique_count[0] = unique_total;
                    a.expanded_count[0] = true_total;
                    a.prefix_tx_ts[0] = static_cast<std::int64_t>(prefix_t0);
                    a.prefix_tx_ts[1] = static_cast<std::int64_t>(ptx::globaltimer_ns());
                }
            }
            __threadfence_block();
            __syncwarp();
            if (lane == 0) {
                *reinterpret_cast<volatile int*>(&sh->prefix_ready) = 1;
                ptx::mbar_arrive(reinterpret_cast<std::uint64_t*>(&sh->prefix_bar));
                BEP_PROF(kProfPrefixReady);
            }
            // zero padding between expert segments: channel c takes local experts c, c+C, ...
            if (a.do_expand && a.zero_padding && !warp_failed(health)) {
                for (int el = c; el < El; el += C) {
                    for (int row = eoff[el] + ecount[el]; row < eoff[el + 1]; ++row) {
                        if (recv_fp8) {
                            for (int b = lane; b < H; b += 32) recv_bytes[static_cast<std::size_t>(row) * H + b] = 0;
                            if (lane == 0) a.recv_scale[row] = 0.0f;
                        } else {
                            zero_row(recv_bytes + static_cast<std::size_t>(row) * out_row_bytes, H, vec_ok);
                        }
                        if (lane == 0) {
                            a.recv_idx[row] = -1;
                            a.recv_w[row] = 0.0f;
                        }
                        if (lane < 3) a.source_meta[static_cast<std::size_t>(row) * 3 + lane] = -1;
                    }
                }
            }
        } else if (lane == 0) {
            // no prefix: release the receive warps all the same (prefix_ready stays 0 and tells them to leave)
            ptx::mbar_arrive(reinterpret_cast<std::uint64_t*>(&sh->prefix_bar));
        }
    } else if (S == 0 && warp <= tx_warps) {
        // ===== send (inside the channel CTA) =====
        const int w = warp - 1;
        if (!use_tma) send_role_vector<kCtaThreads>(k, w, health, st);
        else if (k.stages >= 4) send_role_bulk<4, kCtaThreads>(k, w, health, st);
        else if (k.stages == 3) send_role_bulk<3, kCtaThreads>(k, w, health, st);
        else send_role_bulk<2, kCtaThreads>(k, w, health, st);
        if (lane == 0) atomicMax(&sh->last_tx_ns, ptx::globaltimer_ns());
        if (w == 0 && lane == 0) BEP_PROF(kProfTxDone);
    } else {
        // ===== receive + expand =====
        const int rw = warp - 1 - (S == 0 ? tx_warps : 0);
        if (rw < rx_warps) receive_role<kCtaThreads>(k, rw, health, st);
    }

    // ---- epilogue ----------------------------------------------------------------------------------
    __syncwarp();
    if (lane == 0) {
        if (use_tma) ptx::bulk_wait_all();
        atomicAdd(&sh->stat[kStatSourceTokens], st.source);
        atomicAdd(&sh->stat[kStatRemoteRows], st.remote_rows);
        atomicAdd(&sh->stat[kStatDeliveries], st.deliveries);
        atomicAdd(&sh->stat[kStatEarlyRows], st.early);
        atomicAdd(&sh->stat[kStatRxEmptyProbes], st.probes);
        atomicAdd(&sh->stat[kStatCreditMisses], st.credit);
        atomicAdd(&sh->stat[kStatLocalRows], st.local);
        atomicAdd(&sh->stat[kStatRowsPublished], st.published);
    }
    __syncthreads();
    if (warp == 0) {
        unsigned long long old = 0;
        if (lane == 0) {
            const unsigned long long t_end = ptx::globaltimer_ns();
            prof[kProfEnd] = static_cast<std::int64_t>(t_end);
            std::int64_t* cs = rc->chan_stats + static_cast<std::size_t>(c) * 10;
            for (int i = 0; i < 8; ++i) cs[i] = static_cast<std::int64_t>(sh->stat[i]);
            cs[8] = static_cast<std::int64_t>(t_start);
            cs[9] = static_cast<std::int64_t>(t_end);
            a.prefix_tx_ts[(c + 1) * 2 + 0] = static_cast<std::int64_t>(sh->first_tx_ns);
            a.prefix_tx_ts[(c + 1) * 2 + 1] = static_cast<std::int64_t>(sh->last_tx_ns);
            __threadfence();
            old = atomicAdd(&rc->done_ctas[0], 1ull);
        }
        old = __shfl_sync(full, old, 0);
        if ((old + 1) % static_cast<unsigned long long>(gridDim.x) == 0) {
            // last CTA of this rank: sum the per-CTA statistics (a lane per CTA, then across the warp), hand the
            // staging area back to every source, advance the epoch
            __threadfence();
            std::int64_t sum[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            std::int64_t first = INT64_MAX, last = 0;
            for (int c2 = lane; c2 < static_cast<int>(gridDim.x); c2 += 32) {
                const std::int64_t* o = rc->chan_stats + static_cast<std::size_t>(c2) * 10;
                std::int64_t v[10];
#pragma unroll
                for (int i = 0; i < 10; ++i) v[i] = __ldcg(o + i);
#pragma unroll
                for (int i = 0; i < 8; ++i) sum[i] += v[i];
                first = min(first, v[8]);
                last = max(last, v[9]);
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
                for (int i = 0; i < 8; ++i) sum[i] += __shfl_xor_sync(full, sum[i], o);
                first = min(first, __shfl_xor_sync(full, first, o));
                last = max(last, __shfl_xor_sync(full, last, o));
            }
            if (lane < 8) {
                std::int64_t mine = sum[0];
#pragma unroll
                for (int i = 1; i < 8; ++i)
                    if (static_cast<int>(lane) == i) mine = sum[i];
                a.stats[lane] = mine;
            }
            if (lane == 0) {
                a.timestamps[0] = first;
                a.timestamps[1] = last;
            }
            if (!warp_failed(health)) {
                // The P flags go out side by side, one lane each.  A publishing lane first reads the CTA counter itself
                // (acquire): that orders every CTA's reads of the staging area before this lane's release, which the
                // shuffle that told it the count does not.
                if (lane < static_cast<unsigned>(P) && static_cast<int>(lane) != rc->test_skip_done_to) {
                    (void)ptx::ld_acquire_gpu(reinterpret_cast<const std::uint64_t*>(&rc->done_ctas[0]));
                    ptx::st_release_sys(flag_ptr(rc->seg[lane], lay.done_off, me), epoch);
                }
            }
            __syncwarp();
            if (lane == 0) {
                rc->epochs[0] = epoch;
                if (!a.cached) {  // the layout's running sums change sides (see the layout phase)
                    const int groups = (C + kHistGroup - 1) / kHistGroup;
                    rc->block_hist[static_cast<std::size_t>(C) * (E + P) + static_cast<std::size_t>(2) * (groups + 1) * (E + P)] += 1;
                }
            }
        }
    }
#undef BEP_PROF
#undef BEP_LAYOUT_MARK
}

#endif  // __CUDACC__

}  // namespace bep
