// The send roles of the dispatch kernel: `send_role_bulk` (rows staged in shared memory and pushed with bulk copies,
// READY flags in batches behind one system-scope fence) and `send_role_vector` (16-byte or scalar register copies).
#pragma once

#include "dispatch_common.cuh"

namespace bep {

#ifdef __CUDACC__

namespace detail {

// ---- send role, bulk-copy engine ----------------------------------------------------------------
// The send warps of a CTA serve the tokens of the channels send_first, send_first + send_stride, ...: one
// channel when they sit inside a channel CTA, several when the CTA is a dedicated sender.  Dedicated senders
// exist because an SM with remote stores in flight loses most of its local store throughput (the stores share
// one path out of the SM and the slow ones hold up the fast ones): a few SMs saturate NVLink, so all remote
// stores are confined to those and the channel CTAs' expansion writes run at full HBM speed.  The price is that
// every load of a sender SM is slow too, so the role is built to need few of them and never to wait for one
// row at a time:
//   * routing metadata is fetched for 32 candidate tokens at once (lane = candidate: mask, slot per destination,
//     expert / ordinal / weight per top-k slot; all loads of a batch are in flight together) and parked in a
//     shared-memory tile, from which a row's values are picked up when its turn comes;
//   * payloads run S - 1 rows ahead through a ring of S shared-memory buffers (row n lives in buffer n % S; a
//     buffer is refilled once the outgoing copies of its previous row have finished reading it);
//   * a row's READY flags are stored at least kFlagLag rows late, when its own bulk group has completed, together
//     with those of up to kFlagBatch rows behind one system-scope fence.
//
// Ordering of a row and its READY flag.  The payload leaves through the asynchronous proxy
// (cp.async.bulk shared -> peer global), all copies of one row in one bulk group of the issuing lane.
// `cp.async.bulk.wait_group N` returns to that lane when every group but the N most recent is complete.  That is a
// statement about what the issuing thread can see; it is not a system-scope release.  So before any READY flag goes out
// the issuing lane executes `fence.acq_rel.sys`, then `__syncwarp()` hands the order to the destinations' lanes,
// which store the flags (`st.relaxed.sys`).  (In the conservative setting every lane executes the fence after the
// `__syncwarp()` instead, so that the fence and the flag store it orders are in one thread.)  On this hardware such a
// fence waits for every store the SM still has
// on the wire (measured: 4.4 us when it is paid for every row, against 0.07 us for a flag without it), which is why it
// is not paid per row: the flags of up to kFlagBatch rows wait in registers and go out behind one fence.  A version
// that relied on the completion of the bulk group alone passed the two-GPU litmus and every two-GPU run, and then
// delivered rows whose payload was partly stale on four GPUs with BF16 rows (the flag and the last packets of its row
// took different ways through the switch); the per-row sequence words did not catch it because they sit in the
// row's last bytes.  The receiver reads the flag with `ld.acquire.sys` and issues `fence.proxy.async` before it
// reads the row through the asynchronous proxy.
template <int S, int kCtaThreads>
__device__ __noinline__ void send_role_bulk(const Ctx& k, int w, const Health& cta_health, RoleStats& cta_stats) {
    // own copies: the kernel's objects live in local memory, and every access through a reference is a load or store there
    Health health = cta_health;
    RoleStats st;
    constexpr int D = S - 1;  // rows whose payload is loaded ahead of the one being sent
    static_assert(S >= 2 && S <= kMaxSendStages, "2..4 send stages");
    const DispatchArgs& a = *k.a;
    const RankConst* rc = k.rc;
    const SegmentLayout& lay = k.lay;  // the CTA's copy in shared memory
    const std::uint64_t* const plan_flags = rc->plan_flags;
    const unsigned lane = ptx::lane_id();
    const unsigned full = 0xffffffffu;
    // Every bulk copy of this warp is issued, committed and awaited by lane 31, which never stores a flag
    // (flags belong to lanes 0..P-1).
    const bool issuer = lane == 31u;
    // Segments in registered host memory: completion of a bulk group does not mean its writes have reached host
    // memory (they are posted over PCIe), so there the issuing lane does execute the system-scope fence.
    const bool fence_flags = k.fence_flags;
    const bool fence_every_lane = k.fence_every_lane;
    const unsigned self_bit = 1u << k.me;
    const bool delayed = w == k.send_warps - 1;
    const int P = k.P, K = k.K;
    const int moff = k.wire_fp8 ? lay.meta_off_fp8 : lay.meta_off;
    const unsigned row_bytes = static_cast<unsigned>(moff + lay.meta_bytes);
    const unsigned payload_bytes = static_cast<unsigned>(k.H) * 2u;
    unsigned char* const base = k.row_buffers + static_cast<std::size_t>(w) * S * k.slot_bytes;
    unsigned long long* const bars = &k.sh->mbar[w * S];
    const int tile_stride = P + 3 * K;  // ints per candidate: slot[P] | expert[K] | ordinal[K] | weight[K]
    int* const tile = k.send_tiles + static_cast<std::size_t>(w) * 32 * tile_stride;
    const std::uint32_t seq_epoch = static_cast<std::uint32_t>(k.epoch) + (k.corrupt_sequence ? 1u : 0u);
    BEP_ROLE_DECL();

    // Candidates of this CTA: the tokens of its channels, interleaved; this warp takes every W-th one.
    const int W = k.send_warps;
    const int n_ch = k.send_first < k.C ? (k.C - k.send_first + k.send_stride - 1) / k.send_stride : 0;
    const int n_cand = n_ch * k.Tc;
    int batch = -1;            // batch held in the tile
    unsigned todo = 0;         // candidates of the batch that still have to be sent (bit = lane)
    int my_t = -1, my_ch = 0;  // this lane's candidate of the batch
    unsigned my_mask = 0;
    int issued = 0;            // rows whose payload load has been issued

    // Fetch the routing metadata of candidates w + (32 b + lane) W into the tile.  A dedicated sender reads a plan
    // that another CTA writes in this very launch: a lane first waits for that channel's plan flag.
    auto load_batch = [&](int b) {
        BEP_ROLE_T(t_batch);
        batch = b;
        my_t = -1;
        my_mask = 0u;
        const int ql = w + (b * 32 + static_cast<int>(lane)) * W;
        if (ql < n_cand) {
            // candidates go round the CTA's channels (candidate q = token q / n_ch of channel q % n_ch), so that every
            // channel's receiver sees rows from the start instead of one channel after the other
            const int i = ql % n_ch;
            my_ch = k.send_first + i * k.send_stride;
            const int t = my_ch * k.Tc + ql / n_ch;
            if (t < k.T) {
                bool plan_there = true;
                if (!a.cached && k.plan_is_foreign) {
                    const std::uint64_t* plan_flag = plan_flags + my_ch;
                    while (ptx::ld_acquire_gpu(plan_flag) != k.epoch) {
                        if (health.give_up(kErrGridBarrier, my_ch, 1)) {
                            plan_there = false;
                            break;
                        }
                    }
                }
                if (plan_there) my_t = t;  // (the caller has looked at the failure latch before asking for a batch)
            }
        }
        __syncwarp();  // the tile's previous contents have been picked up by every lane
        if (my_t >= 0) {
            int* row = tile + static_cast<int>(lane) * tile_stride;
            const int t = my_t;
            // Everything the first eight ranks and the first eight choices need is requested before anything is
            // used: one round trip to memory per batch, also for the destination mask (slots of ranks the token
            // does not go to are stored as -1 in the plan, so they need no mask to be read).
            const unsigned raw_mask = a.plan_mask[t];
            int slot8[8], ord8[8];
            std::int64_t e8[8];
            float w8[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) slot8[u] = u < P ? a.plan_slot[static_cast<std::size_t>(t) * P + u] : -1;
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const bool in = u < K;
                const std::size_t at = static_cast<std::size_t>(t) * K + (in ? u : 0);
                e8[u] = in ? a.topk_idx[at] : -1;
                ord8[u] = in ? a.plan_expert_ord[at] : -1;
                w8[u] = (in && a.topk_w) ? a.topk_w[at] : 1.0f;
            }
            my_mask = raw_mask & ~self_bit;
            if (my_mask != 0u) {
#pragma unroll
                for (int u = 0; u < 8; ++u)
                    if (u < P) row[u] = (my_mask >> u & 1u) ? slot8[u] : -1;
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    if (u < K) {
                        row[P + u] = (e8[u] >= 0 && e8[u] < k.E) ? static_cast<int>(e8[u]) : -1;
                        row[P + K + u] = ord8[u];
                        row[P + 2 * K + u] = __float_as_int(w8[u]);
                    }
                }
                for (int d = 8; d < P; ++d) row[d] = (my_mask >> d & 1u) ? a.plan_slot[static_cast<std::size_t>(t) * P + d] : -1;
                for (int kk = 8; kk < K; ++kk) {
                    const std::size_t at = static_cast<std::size_t>(t) * K + kk;
                    const std::int64_t e = a.topk_idx[at];
                    row[P + kk] = (e >= 0 && e < k.E) ? static_cast<int>(e) : -1;
                    row[P + K + kk] = a.plan_expert_ord[at];
                    row[P + 2 * K + kk] = __float_as_int(a.topk_w ? a.topk_w[at] : 1.0f);
                }
            }
        }
        __syncwarp();
        todo = __ballot_sync(full, my_mask != 0u);
        BEP_ROLE_ADD(kRoleMetaNs, t_batch);
        BEP_ROLE_MARK(kRoleFirstBatchNs);
    };

    // Next row to send: picks its metadata out of the tile and issues its payload load.
    auto next_token = [&](TokenRegs& r) -> bool {
        while (todo == 0u) {
            const int b = batch + 1;
            if (w + b * 32 * W >= n_cand || warp_failed(health)) return false;
            load_batch(b);
        }
        const int src = __ffs(todo) - 1;
        todo &= todo - 1;
        r.t = __shfl_sync(full, my_t, src);
        r.ch = __shfl_sync(full, my_ch, src);
        r.mask = __shfl_sync(full, my_mask, src);
        const int* row = tile + src * tile_stride;
        r.j = lane < static_cast<unsigned>(P) ? row[lane] : -1;
        r.e = -1;
        r.ord = -1;
        r.w = 0.0f;
        if (lane < static_cast<unsigned>(K)) {
            r.e = row[P + lane];
            r.ord = row[P + K + lane];
            r.w = __int_as_float(row[P + 2 * K + lane]);
        }
        // payload into the next buffer of the ring, once the row that used it has been read out of it
        if (issuer) {
            const int b = issued % S;
            bulk_wait_group_read<0>();
            std::uint64_t* bar = reinterpret_cast<std::uint64_t*>(&bars[b]);
            ptx::mbar_expect_tx(bar, payload_bytes);
            ptx::bulk_g2s(base + static_cast<std::size_t>(b) * k.slot_bytes, a.x + static_cast<std::size_t>(r.t) * k.H, payload_bytes, bar);
        }
        ++issued;
        return true;
    };

    TokenRegs ahead[D];
    bool ahead_ok[D];
#pragma unroll
    for (int i = 0; i < D; ++i) ahead_ok[i] = (i == 0 || ahead_ok[i - 1]) ? next_token(ahead[i]) : false;

    // READY flags not yet stored: the newest row's at the end, one step towards the front per row.  A flag may go out
    // once its row's bulk group is complete (all but the kFlagLag most recent groups are, after the wait below) and a
    // system-scope fence has followed; one such fence serves the flags of up to `flag_batch` rows.
    constexpr int kRing = kFlagBatch + kFlagLag;
    std::uint64_t* flag_ring[kRing];
    std::uint32_t flag_seq[kRing];
#pragma unroll
    for (int i = 0; i < kRing; ++i) {
        flag_ring[i] = nullptr;
        flag_seq[i] = 0;
    }
    // rows per fence: every row on host segments (as before); on peer segments a quarter of what this warp has to
    // send, at most kFlagBatch, so that a warp with a handful of rows does not sit on their flags
    const int flag_batch = fence_flags ? 1 : max(1, min(kFlagBatch, n_cand / (4 * max(W, 1))));
    int since_flags = 0;  // rows issued since flags last went out
    bool first_flags_stamped = false;
    int n = 0;  // rows sent
    bool broke = false;
    while (ahead_ok[0]) {
        const TokenRegs cur = ahead[0];
#pragma unroll
        for (int i = 0; i + 1 < D; ++i) {
            ahead[i] = ahead[i + 1];
            ahead_ok[i] = ahead_ok[i + 1];
        }
        ahead_ok[D - 1] = ahead_ok[D - 1] ? next_token(ahead[D - 1]) : false;
#if BEP_ENABLE_PROFILING
        {   // the issuing lane may sit in next_token's buffer wait: make the warp's wait show up under a name of its own
            BEP_ROLE_T(t_buffer);
            __syncwarp();
            BEP_ROLE_ADD(kRoleBufferWaitNs, t_buffer);
        }
#endif

        unsigned char* buf = base + static_cast<std::size_t>(n % S) * k.slot_bytes;
        const unsigned parity = static_cast<unsigned>(n / S) & 1u;
        // destination row of lane d
        std::uint8_t* dst = nullptr;
        std::uint64_t* ready = nullptr;
        if (cur.j >= 0) {
            const std::size_t ring_index = (static_cast<std::size_t>(k.me) * k.C + cur.ch) * k.Q + (cur.j % k.Q);
            dst = k.seg[lane] + lay.stage_off + ring_index * lay.row_stride;
            ready = reinterpret_cast<std::uint64_t*>(k.seg[lane] + lay.ready_off) + ring_index;
        }
        if (k.ring) {
            // Bounded rings: slot j % Q is free once the receiver has acknowledged row j - Q.  The receiver only
            // sees rows whose READY flags are out, so before this warp settles down to wait for credit it
            // stores every flag it still holds back.
            BEP_ROLE_T(t_credit);
            const bool need = cur.j >= k.Q;
            const std::uint64_t* ack = nullptr;
            std::uint64_t want = 0;
            bool have = true;
            if (need) {
                ack = reinterpret_cast<const std::uint64_t*>(k.my_seg + lay.ack_off) +
                      (static_cast<std::size_t>(lane) * k.C + cur.ch) * k.Q + (cur.j % k.Q);
                want = make_seq(k.epoch, static_cast<std::uint32_t>(cur.j - k.Q + 1));
                have = ptx::ld_acquire_sys(ack) == want;
            }
            if (!__all_sync(full, have)) {
                if (issuer) {
                    bulk_wait_group<0>();
                    if (!fence_every_lane) ptx::fence_sys();
                }
                __syncwarp();
                if (fence_every_lane) ptx::fence_sys();  // (see the note on the two chains below)
#pragma unroll
                for (int i = 0; i < kRing; ++i) {
                    if (flag_ring[i] != nullptr) ptx::st_relaxed_sys(flag_ring[i], make_seq(k.epoch, flag_seq[i]));
                    flag_ring[i] = nullptr;
                }
                since_flags = 0;
                if (!have) {
                    ++st.credit;
                    while (ptx::ld_acquire_sys(ack) != want) {
                        if (health.give_up(kErrCreditWait, lane, cur.j)) break;
                    }
                }
            }
            BEP_ROLE_ADD(kRoleCreditWaitNs, t_credit);
        }
        __syncwarp();
        // The failure latch lives in global memory and a load is slow on an SM that is busy storing to peers: it is
        // looked at every eighth row here (every bounded wait looks at it as well).
        if ((n & 7) == 0 && warp_failed(health)) {
            broke = true;
            break;
        }
        if (delayed) test_delay(k.delay_meta_ns);
        // BF16 wire: the metadata lies behind the payload and can be written while the payload is still landing
        if (!k.wire_fp8) write_row_meta(buf + moff, lay, cur.t, 1.0f, seq_epoch, cur.e, cur.ord, cur.w, K);
        BEP_ROLE_T(t_load);
        const bool arrived = mbar_wait_bounded(&bars[n % S], parity, health);
        BEP_ROLE_ADD(kRoleLoadWaitNs, t_load);
        if (!__all_sync(full, arrived)) {
            broke = true;
            break;
        }
        if (lane == 0 && k.sh->first_tx_ns == 0) atomicCAS(&k.sh->first_tx_ns, 0ull, ptx::globaltimer_ns());
        if (delayed) test_delay(k.delay_tx_ns);
        if (k.wire_fp8) {
            BEP_ROLE_T(t_quant);
            const float scale = quantise_row_in_place(buf, k.H);
            write_row_meta(buf + moff, lay, cur.t, scale, seq_epoch, cur.e, cur.ord, cur.w, K);
            BEP_ROLE_ADD(kRoleQuantNs, t_quant);
        }
        BEP_ROLE_T(t_issue);
        ptx::fence_proxy_async_smem();
        __syncwarp();
        for (unsigned m = cur.mask; m; m &= m - 1) {
            std::uint8_t* d = shfl_ptr(dst, __ffs(m) - 1);
            if (issuer) ptx::bulk_s2g(d, buf, row_bytes);
        }
        if (issuer) ptx::bulk_commit();
        BEP_ROLE_ADD(kRoleIssueNs, t_issue);
        BEP_ROLE_MARK(kRoleFirstIssueNs);
        // this row's flags join the ring (an entry that reaches the front has long been stored: flags go out at
        // least every kFlagBatch rows and the ring holds kFlagBatch + kFlagLag)
#pragma unroll
        for (int i = 0; i + 1 < kRing; ++i) {
            flag_ring[i] = flag_ring[i + 1];
            flag_seq[i] = flag_seq[i + 1];
        }
        flag_ring[kRing - 1] = ready;
        flag_seq[kRing - 1] = static_cast<std::uint32_t>(cur.j + 1);
        ++since_flags;
        // READY flags of every row but the kFlagLag most recent: their bulk groups are complete after the wait, and
        // the fence that follows orders those writes before the flags at system scope.  (Completion of a bulk group
        // alone is not enough: it tells this thread that the writes are done as far as it can see, and with four
        // ranks and BF16 rows a relaxed flag was seen to overtake part of its row on its way through the switch.)
        // Two chains.  By default the issuing lane fences and the warp barrier carries the order to the lanes that
        // store the flags (one fence instruction with one active lane; what the litmus and the payload checks ran).
        // In the conservative setting (`fence_every_lane`, one fence per row as well) every lane fences after the
        // barrier, so that the fence and the flag store it orders are in the same thread: the release pattern as the
        // memory model spells it.
        if (since_flags >= flag_batch && n >= kFlagLag) {
            BEP_ROLE_T(t_store);
            if (issuer) {
                bulk_wait_group<kFlagLag>();
                if (!fence_every_lane) ptx::fence_sys();
            }
            __syncwarp();
            if (fence_every_lane) ptx::fence_sys();
#pragma unroll
            for (int i = 0; i < kRing - kFlagLag; ++i) {
                if (flag_ring[i] != nullptr) ptx::st_relaxed_sys(flag_ring[i], make_seq(k.epoch, flag_seq[i]));
                flag_ring[i] = nullptr;
            }
            since_flags = 0;
            BEP_ROLE_ADD(kRoleStoreWaitNs, t_store);
            if (w == 0 && lane == 0 && !first_flags_stamped) k.prof[kProfFirstTxDone] = static_cast<std::int64_t>(ptx::globaltimer_ns());
            first_flags_stamped = true;
        }
        if (lane == 0) {
            ++st.source;
            st.deliveries += __popc(cur.mask);
            st.published += __popc(cur.mask);
            if (*reinterpret_cast<volatile int*>(&k.sh->prefix_ready) == 0) ++st.early;
        }
        BEP_ROLE_COUNT(kRoleRows, 1);
        ++n;
    }
    // drain: the last rows' groups, then their flags in row order
    {
        BEP_ROLE_T(t_store);
        if (issuer) {
            bulk_wait_group<0>();
            if (!fence_every_lane) ptx::fence_sys();
        }
        __syncwarp();
        if (fence_every_lane) ptx::fence_sys();
        if (!broke && !warp_failed(health)) {
#pragma unroll
            for (int i = 0; i < kRing; ++i)
                if (flag_ring[i] != nullptr) ptx::st_relaxed_sys(flag_ring[i], make_seq(k.epoch, flag_seq[i]));
            if (w == 0 && lane == 0 && n > 0 && !first_flags_stamped) k.prof[kProfFirstTxDone] = static_cast<std::int64_t>(ptx::globaltimer_ns());
        }
        BEP_ROLE_ADD(kRoleStoreWaitNs, t_store);
        BEP_ROLE_ADD(kRoleDrainNs, t_store);
    }
    // a failed warp leaves with loads still on their way into its buffers: give them a bounded time to land
    for (int r = n; r < issued; ++r) {
        unsigned polls = 0;
        while (!ptx::mbar_try_wait(reinterpret_cast<std::uint64_t*>(&bars[r % S]), static_cast<unsigned>(r / S) & 1u) && ++polls < (1u << 20))
            ptx::nanosleep(64);
    }
    cta_stats = st;
    BEP_ROLE_FLUSH(k.role_prof ? k.role_prof + static_cast<std::size_t>(threadIdx.x >> 5) * kRoleFields : nullptr);
}

// ---- send role, register path (16-byte or scalar accesses; also the path for odd hidden sizes) ----
template <int kCtaThreads>
__device__ __noinline__ void send_role_vector(const Ctx& k, int w, const Health& cta_health, RoleStats& cta_stats) {
    // own copies: the kernel's objects live in local memory, and every access through a reference is a load or store there
    Health health = cta_health;
    RoleStats st;
    const DispatchArgs& a = *k.a;
    const RankConst* rc = k.rc;
    const SegmentLayout& lay = k.lay;  // the CTA's copy in shared memory
    const std::uint64_t* const plan_flags = rc->plan_flags;
    const unsigned lane = ptx::lane_id();
    const unsigned self_bit = 1u << k.me;
    const bool delayed = w == k.send_warps - 1;
    unsigned char* meta_sm = k.sh->meta[threadIdx.x >> 5];
    const std::uint32_t seq_epoch = static_cast<std::uint32_t>(k.epoch) + (k.corrupt_sequence ? 1u : 0u);
    const int moff = k.wire_fp8 ? lay.meta_off_fp8 : lay.meta_off;
    BEP_ROLE_DECL();
    int sent = 0;
    const int n_ch = k.send_first < k.C ? (k.C - k.send_first + k.send_stride - 1) / k.send_stride : 0;
    const int n_cand = n_ch * k.Tc;
    for (int q = w; q < n_cand; q += k.send_warps) {
        if (warp_failed(health)) break;
        const int ch = k.send_first + (q % n_ch) * k.send_stride;  // round the CTA's channels
        const int t = ch * k.Tc + q / n_ch;
        if (t >= k.T) continue;
        if (!a.cached && k.plan_is_foreign) {
            // a dedicated sender reads a plan that the channel's own CTA writes in this launch
            if (lane == 0) {
                const std::uint64_t* plan_flag = plan_flags + ch;
                while (ptx::ld_acquire_gpu(plan_flag) != k.epoch) {
                    if (health.give_up(kErrGridBarrier, ch, 1)) break;
                }
            }
            __syncwarp();
            if (warp_failed(health)) break;
        }
        const unsigned mask = a.plan_mask[t] & ~self_bit;
        if (mask == 0) continue;
        int j = -1;
        std::uint8_t* dst = nullptr;
        std::uint64_t* ready = nullptr;
        if (lane < static_cast<unsigned>(k.P) && (mask >> lane & 1u)) {
            j = a.plan_slot[static_cast<std::size_t>(t) * k.P + lane];
            const std::size_t ring_index = (static_cast<std::size_t>(k.me) * k.C + ch) * k.Q + (j % k.Q);
            dst = k.seg[lane] + lay.stage_off + ring_index * lay.row_stride;
            ready = reinterpret_cast<std::uint64_t*>(k.seg[lane] + lay.ready_off) + ring_index;
            if (k.ring && j >= k.Q) {
                const std::uint64_t* ack = reinterpret_cast<const std::uint64_t*>(k.my_seg + lay.ack_off) +
                                           (static_cast<std::size_t>(lane) * k.C + ch) * k.Q + (j % k.Q);
                const std::uint64_t want = make_seq(k.epoch, static_cast<std::uint32_t>(j - k.Q + 1));
                bool missed = false;
                while (ptx::ld_acquire_sys(ack) != want) {
                    missed = true;
                    if (health.give_up(kErrCreditWait, lane, j)) break;
                }
                if (missed) ++st.credit;
            }
        }
        __syncwarp();
        if (warp_failed(health)) break;
        const std::uint8_t* src = reinterpret_cast<const std::uint8_t*>(a.x + static_cast<std::size_t>(t) * k.H);
        if (delayed) test_delay(k.delay_meta_ns);
        int e, ord;
        float wt;
        load_token_routes(a, t, k.K, k.E, e, ord, wt);
        if (lane == 0 && k.sh->first_tx_ns == 0) atomicCAS(&k.sh->first_tx_ns, 0ull, ptx::globaltimer_ns());
        if (delayed) test_delay(k.delay_tx_ns);
        float scale = 1.0f;
        if (k.wire_fp8) scale = tx_row_fp8(src, dst, mask, -1, k.H, k.vec_ok);
        else tx_row_bf16(src, dst, mask, k.H, k.vec_ok);
        write_row_meta(meta_sm, lay, t, scale, seq_epoch, e, ord, wt, k.K);
        __syncwarp();
        for (unsigned m = mask; m; m &= m - 1) {
            std::uint8_t* mdst = shfl_ptr(dst, __ffs(m) - 1) + moff;
            for (int q = lane; q < lay.meta_bytes / 16; q += 32)
                ptx::st_v4(mdst + q * 16, *reinterpret_cast<const uint4*>(meta_sm + q * 16));
        }
        // every lane's stores, then the warp joins, then one lane per destination releases that row's flag
        __syncwarp();
        if (j >= 0) ptx::st_release_sys(ready, make_seq(k.epoch, static_cast<std::uint32_t>(j + 1)));
        if (lane == 0) {
            ++st.source;
            st.deliveries += __popc(mask);
            st.published += __popc(mask);
            if (*reinterpret_cast<volatile int*>(&k.sh->prefix_ready) == 0) ++st.early;
            if (w == 0 && sent == 0) k.prof[kProfFirstTxDone] = static_cast<std::int64_t>(ptx::globaltimer_ns());
        }
        BEP_ROLE_COUNT(kRoleRows, 1);
        ++sent;
    }
    cta_stats = st;
    BEP_ROLE_FLUSH(k.role_prof ? k.role_prof + static_cast<std::size_t>(threadIdx.x >> 5) * kRoleFields : nullptr);
}

}  // namespace detail

#endif  // __CUDACC__

}  // namespace bep
