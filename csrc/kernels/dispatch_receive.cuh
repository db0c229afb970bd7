// The receive + expand role of the dispatch kernel.
#pragma once

#include "dispatch_common.cuh"

namespace bep {

#ifdef __CUDACC__

namespace detail {

// ---- receive + expand role ------------------------------------------------------------------------
// Remote rows: poll the READY flags of this channel's rings (local memory), read a staged row once, check its
// sequence words, write it to its output rows.  Own rows: whenever no remote row is waiting, take the next own
// token that has a local expert straight from `x`.
template <int kCtaThreads>
__device__ __noinline__ void receive_role(const Ctx& k, int w, const Health& cta_health, RoleStats& cta_stats) {
    // own copies: the kernel's objects live in local memory, and every access through a reference is a load or store there
    Health health = cta_health;
    RoleStats st;
    const DispatchArgs& a = *k.a;
    const RankConst* rc = k.rc;
    const SegmentLayout& lay = k.lay;  // the CTA's copy in shared memory
    const unsigned lane = ptx::lane_id();
    const unsigned full = 0xffffffffu;
    const bool delayed = w == k.rx_warps - 1;
    const int P = k.P, C = k.C, Q = k.Q, K = k.K, H = k.H, me = k.me, c = k.c;
    BEP_ROLE_DECL();
    // The control warp owns the diagnosis of a missing counts message (it knows which source is late); this
    // wait only has to end, so its own deadline is a quarter of the timeout later.
    health.deadline += k.timeout_ns / 4;
    {
        // The wait sits on an mbarrier: a waiting warp is suspended by the hardware instead of taking issue slots from
        // the control warp that it is waiting for.
        BEP_ROLE_T(t_prefix);
        while (!ptx::mbar_try_wait(reinterpret_cast<std::uint64_t*>(&k.sh->prefix_bar), 0u)) {
            if (warp_give_up(health, kErrCountsWait, -1, 0)) break;
        }
        BEP_ROLE_ADD(kRolePrefixWaitNs, t_prefix);
    }
    __threadfence_block();
    __syncwarp();
    if (!warp_failed(health) && *reinterpret_cast<volatile int*>(&k.sh->prefix_ready) != 0) {
        int next_j = w;
        // rows of this rank itself do not come through the ring
        const int expect = (lane < static_cast<unsigned>(P) && static_cast<int>(lane) != me) ? k.sh->chan_expected[lane] : 0;
        int t_local = k.t0 + w;
        const std::uint64_t* ready_base = reinterpret_cast<const std::uint64_t*>(k.my_seg + lay.ready_off);
        const int buffer_index = k.rx_buffer_base + w;
        unsigned char* my_slot = k.row_buffers + static_cast<std::size_t>(buffer_index) * k.slot_bytes;
        unsigned long long* my_bar = &k.sh->mbar[buffer_index];
        unsigned parity = 0;
        bool stop = false;
        while (!stop) {
            const bool pending = next_j < expect;
            const unsigned pend = __ballot_sync(full, pending);
            if (pend == 0 && t_local >= k.t1) break;
            bool hit = false;
            if (pending) {
                const std::uint64_t v = ptx::ld_acquire_sys(ready_base + (static_cast<std::size_t>(lane) * C + c) * Q + (next_j % Q));
                hit = v == make_seq(k.epoch, static_cast<std::uint32_t>(next_j + 1));
            }
            const unsigned hits = __ballot_sync(full, hit);
            // the acquiring lane's observation is ordered before every lane's reads of the row
            __syncwarp();
            if (hits == 0 && t_local < k.t1) {
                // ---- one own token, straight from x ----
                const int t = t_local;
                t_local += k.rx_warps;
                const unsigned mask = a.plan_mask[t];
                if ((mask >> me & 1u) == 0) continue;
                const int j = a.plan_slot[static_cast<std::size_t>(t) * P + me];
                int e, ord;
                float wgt;
                load_token_routes(a, t, K, k.E, e, ord, wgt);
                const std::uint8_t* src = reinterpret_cast<const std::uint8_t*>(a.x + static_cast<std::size_t>(t) * H);
                std::uint8_t* out_ptr = nullptr;
                int n_rows = 0;
                if (k.use_tma) {
                    BEP_ROLE_T(t_drain);
                    if (lane == 0) {
                        ptx::bulk_wait_read_all();  // the previous row's stores have left the buffer
                        ptx::mbar_expect_tx(reinterpret_cast<std::uint64_t*>(my_bar), static_cast<unsigned>(H) * 2u);
                        ptx::bulk_g2s(my_slot, src, static_cast<unsigned>(H) * 2u, reinterpret_cast<std::uint64_t*>(my_bar));
                    }
                    BEP_ROLE_ADD(kRoleStoreWaitNs, t_drain);
                    BEP_ROLE_T(t_load);
                    const bool arrived = mbar_wait_bounded(my_bar, parity, health);
                    parity ^= 1u;
                    BEP_ROLE_ADD(kRoleLoadWaitNs, t_load);
                    if (!__all_sync(full, arrived)) break;
                    float scale = 1.0f;
                    if (k.recv_fp8) {
                        scale = quantise_row_in_place(my_slot, H);
                        ptx::fence_proxy_async_smem();
                        __syncwarp();
                    }
                    BEP_ROLE_T(t_meta);
                    const bool overflow = place_row(k, me, j, t, scale, e, ord, wgt, out_ptr, n_rows);
                    BEP_ROLE_ADD(kRoleMetaNs, t_meta);
                    if (overflow) {
                        if (lane == 0) record_error(rc, a.error, kErrCapacity, me, j);
                        break;
                    }
                    if (delayed) test_delay(k.delay_scatter_ns);
                    for (int i = 0; i < n_rows; ++i) {
                        std::uint8_t* dst = shfl_ptr(out_ptr, i);
                        if (lane == 0) ptx::bulk_s2g(dst, my_slot, static_cast<unsigned>(k.out_row_bytes));
                    }
                    if (lane == 0) ptx::bulk_commit();
                } else {
                    const float scale = k.recv_fp8 ? row_scale_from_global(src, H, k.vec_ok) : 1.0f;
                    const bool overflow = place_row(k, me, j, t, scale, e, ord, wgt, out_ptr, n_rows);
                    if (overflow) {
                        if (lane == 0) record_error(rc, a.error, kErrCapacity, me, j);
                        break;
                    }
                    if (delayed) test_delay(k.delay_scatter_ns);
                    if (k.recv_fp8) tx_row_fp8(src, out_ptr, n_rows >= 32 ? full : (1u << n_rows) - 1u, -1, H, k.vec_ok);
                    else rx_row_scatter(src, false, 1.0f, out_ptr, n_rows, H, k.vec_ok);
                }
                if (lane == 0) ++st.local;
                BEP_ROLE_COUNT(kRoleLocalRows, 1);
                BEP_ROLE_COUNT(kRoleRows, 1);
                continue;
            }
            if (hits == 0) {
                BEP_ROLE_T(t_idle);
                ++st.probes;
                const bool give_up = warp_give_up(health, kErrRowWait, __ffs(pend) - 1, 0);
                BEP_ROLE_ADD(kRoleIdlePollNs, t_idle);
                if (give_up) break;
                continue;
            }
            for (unsigned hm = hits; hm && !stop; hm &= hm - 1) {
                const int s = __ffs(hm) - 1;
                const int j = __shfl_sync(full, next_j, s);
                if (lane == static_cast<unsigned>(s)) next_j += k.rx_warps;
                const bool fp8row = k.wire_fp8;
                const std::size_t ring_index = (static_cast<std::size_t>(s) * C + c) * Q + (j % Q);
                const std::uint8_t* row_src = k.my_seg + lay.stage_off + ring_index * lay.row_stride;
                const int moff = fp8row ? lay.meta_off_fp8 : lay.meta_off;
                if (delayed) test_delay(k.delay_rx_ns);
                const unsigned char* meta;
                if (k.use_tma) {
                    ptx::fence_proxy_async();
                    BEP_ROLE_T(t_drain);
                    if (lane == 0) {
                        const unsigned bytes = static_cast<unsigned>(moff + lay.meta_bytes);
                        ptx::bulk_wait_read_all();  // the previous row's stores have left the buffer
                        ptx::mbar_expect_tx(reinterpret_cast<std::uint64_t*>(my_bar), bytes);
                        ptx::bulk_g2s(my_slot, row_src, bytes, reinterpret_cast<std::uint64_t*>(my_bar));
                    }
                    BEP_ROLE_ADD(kRoleStoreWaitNs, t_drain);
                    BEP_ROLE_T(t_load);
                    const bool arrived = mbar_wait_bounded(my_bar, parity, health);
                    parity ^= 1u;
                    BEP_ROLE_ADD(kRoleLoadWaitNs, t_load);
                    if (!__all_sync(full, arrived)) {
                        stop = true;
                        break;
                    }
                    meta = my_slot + moff;
                } else {
                    meta = row_src + moff;
                }
                BEP_ROLE_T(t_meta);
                // metadata -> registers
                int token, seq_epoch, seq_index;
                float scale;
                if (k.use_tma) {
                    token = reinterpret_cast<const int*>(meta)[0];
                    scale = reinterpret_cast<const float*>(meta)[1];
                    seq_epoch = reinterpret_cast<const int*>(meta)[2];
                    seq_index = reinterpret_cast<const int*>(meta)[3];
                } else {
                    token = ptx::ld_volatile(reinterpret_cast<const int*>(meta));
                    scale = __int_as_float(ptx::ld_volatile(reinterpret_cast<const int*>(meta) + 1));
                    seq_epoch = ptx::ld_volatile(reinterpret_cast<const int*>(meta) + 2);
                    seq_index = ptx::ld_volatile(reinterpret_cast<const int*>(meta) + 3);
                }
                int e = -1, ord = 0;
                float wgt = 0.0f;
                if (lane < static_cast<unsigned>(K)) {
                    const int* mi = reinterpret_cast<const int*>(meta + 16);
                    if (k.use_tma) {
                        e = mi[lane];
                        ord = mi[K + lane];
                        wgt = __int_as_float(mi[2 * K + lane]);
                    } else {
                        e = ptx::ld_volatile(mi + lane);
                        ord = ptx::ld_volatile(mi + K + lane);
                        wgt = __int_as_float(ptx::ld_volatile(mi + 2 * K + lane));
                    }
                }
                __syncwarp();
                // the payload behind a READY flag must be the one of this epoch and of the token its header names
                if (static_cast<std::uint32_t>(seq_epoch) != static_cast<std::uint32_t>(k.epoch) ||
                    static_cast<std::uint32_t>(seq_index) != static_cast<std::uint32_t>(token) + 1u || token < 0 ||
                    token >= lay.num_max_tokens) {
                    if (lane == 0) record_error(rc, a.error, kErrSequence, s, j);
                    stop = true;
                    break;
                }
                std::uint8_t* out_ptr = nullptr;
                int n_rows = 0;
                const bool overflow = place_row(k, s, j, token, scale, e, ord, wgt, out_ptr, n_rows);
                BEP_ROLE_ADD(kRoleMetaNs, t_meta);
                if (overflow) {
                    if (lane == 0) record_error(rc, a.error, kErrCapacity, s, j);
                    stop = true;
                    break;
                }
                if (delayed) test_delay(k.delay_scatter_ns);
                std::uint64_t* ack = reinterpret_cast<std::uint64_t*>(k.seg[s] + lay.ack_off) +
                                     (static_cast<std::size_t>(me) * C + c) * Q + (j % Q);
                if (!k.use_tma) {
                    if (k.recv_fp8) rx_row_copy_bytes(row_src, out_ptr, n_rows, H);
                    else rx_row_scatter(row_src, fp8row, scale, out_ptr, n_rows, H, k.vec_ok);
                    if (k.ring) {
                        __syncwarp();
                        if (lane == 0) ptx::st_release_sys(ack, make_seq(k.epoch, static_cast<std::uint32_t>(j + 1)));
                    }
                } else {
                    // the row is in shared memory (the load has completed): its ring slot can be handed back already;
                    // nothing this lane wrote has to become visible first, so the store carries no fence
                    if (k.ring && lane == 0) ptx::st_relaxed_sys(ack, make_seq(k.epoch, static_cast<std::uint32_t>(j + 1)));
                    if (fp8row && !k.recv_fp8) {
                        BEP_ROLE_T(t_quant);
                        // widen in place, decreasing order: chunk q is read before anything lands on it
                        const int chunks = H / 8;
                        for (int q0 = (chunks - 1) / 32 * 32; q0 >= 0; q0 -= 32) {
                            const int q = q0 + lane;
                            uint2 f = make_uint2(0, 0);
                            if (q < chunks) f = *reinterpret_cast<const uint2*>(my_slot + q * 8);
                            __syncwarp();
                            if (q < chunks) *reinterpret_cast<uint4*>(my_slot + q * 16) = chunk_from_fp8(f, scale);
                            __syncwarp();
                        }
                        ptx::fence_proxy_async_smem();
                        __syncwarp();
                        BEP_ROLE_ADD(kRoleQuantNs, t_quant);
                    }
                    BEP_ROLE_T(t_issue);
                    for (int i = 0; i < n_rows; ++i) {
                        std::uint8_t* dst = shfl_ptr(out_ptr, i);
                        if (lane == 0) ptx::bulk_s2g(dst, my_slot, static_cast<unsigned>(k.out_row_bytes));
                    }
                    if (lane == 0) ptx::bulk_commit();
                    BEP_ROLE_ADD(kRoleIssueNs, t_issue);
                }
                if (lane == 0) ++st.remote_rows;
                BEP_ROLE_COUNT(kRoleRows, 1);
                if (w == 0 && lane == 0 && k.prof[kProfFirstRxRow] == 0) k.prof[kProfFirstRxRow] = static_cast<std::int64_t>(ptx::globaltimer_ns());
            }
        }
        if (w == 0 && lane == 0) k.prof[kProfRxDone] = static_cast<std::int64_t>(ptx::globaltimer_ns());
    }
    cta_stats = st;
    BEP_ROLE_FLUSH(k.role_prof ? k.role_prof + static_cast<std::size_t>(threadIdx.x >> 5) * kRoleFields : nullptr);
}

}  // namespace detail

#endif  // __CUDACC__

}  // namespace bep
