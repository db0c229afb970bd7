// Fused expert-parallel dispatch: one cooperative launch per rank does what the reference spreads
// over eight launches (csrc/buffers/advanced.hpp:472-523): epoch bookkeeping, route validation,
// stable ordinals, counts exchange, the all-to-all itself, receive-side expansion into per-expert
// rows, local-token handling, zero padding and statistics.
//
// Grid: (channels, virtual_ranks).  blockIdx.y picks the rank (more than one only when several
// ranks are emulated on one GPU), blockIdx.x the channel.  Channel c of a rank sends that rank's
// tokens [c*ceil(T/C), (c+1)*ceil(T/C)) and receives what channel c of every rank sent to it.
//
// Warp roles inside a channel CTA (the reference's control / TX / RX / scatter roles,
// csrc/kernels/host_staged/advanced_dispatch.cuh:287-752, fused_receive.cuh:199-305):
//   warp 0              control: reuse guard, stable ordinals, receive prefix, zero padding
//   warps 1..tx         send: read a token row once, (quantise,) store it into the staging ring
//                       of every destination rank, then release that row's READY flag there
//   warps tx+1..        receive+expand: poll READY flags in local memory, read the staged row once
//                       and write it to every local expert row (or the unique row)
//
// Transport: a row crosses NVLink once per (token, destination rank) as posted stores into the
// destination's segment (16-byte stores, or cp.async.bulk from shared memory); every flag is
// written by exactly one rank and polled only by its owner in local memory.
#pragma once

#include "protocol.cuh"
#include "quant.cuh"

namespace bep {

constexpr int kMetaSmemBytes = 16 + 12 * kMaxTopk;

struct DispatchShared {
    int cnt_r[kMaxRanks];
    unsigned bits_r[kMaxRanks];
    int total_r[kMaxRanks];
    int chan_expected[kMaxRanks];
    int chan_base[kMaxRanks];
    int source_offsets[kMaxRanks + 1];
    int prefix_ready;
    int cta_flag;
    unsigned long long stat[8];
    unsigned long long first_tx_ns;
    unsigned long long last_tx_ns;
    unsigned long long mbar[kMaxWarps];
    alignas(16) unsigned char meta[kMaxWarps][kMetaSmemBytes];
};

// Dynamic shared memory: header | cnt_e[E] | bits_e[E] | total_e[E] | eoff[El+1] | ecount[El] |
// spre[P*El] | msg[P*counts_stride] | (TMA only) one row buffer per send/receive warp.
inline std::size_t dispatch_smem_bytes(const SegmentLayout& lay, int tx_warps, int rx_warps, bool use_tma) {
    std::size_t bytes = align_up(sizeof(DispatchShared), 16);
    bytes += static_cast<std::size_t>(lay.num_experts) * 12;
    bytes += static_cast<std::size_t>(lay.num_local_experts) * 8 + 4;
    bytes += static_cast<std::size_t>(lay.num_ranks) * lay.num_local_experts * 4;
    bytes = align_up(bytes, 16) + static_cast<std::size_t>(lay.num_ranks) * lay.counts_stride * 4;
    bytes = align_up(bytes, 128);
    if (use_tma) bytes += static_cast<std::size_t>(tx_warps + rx_warps) * align_up(lay.meta_off + lay.meta_bytes, 128);
    return bytes;
}

#ifdef __CUDACC__

namespace detail {

__device__ __forceinline__ bool cta_failed(const Health& health, int* smem_flag) {
    __syncthreads();
    if (threadIdx.x == 0) *smem_flag = health.failed() ? 1 : 0;
    __syncthreads();
    return *smem_flag != 0;
}

__device__ __forceinline__ std::uint8_t* shfl_ptr(std::uint8_t* p, int src_lane) {
    const unsigned long long v = __shfl_sync(0xffffffffu, reinterpret_cast<unsigned long long>(p), src_lane);
    return reinterpret_cast<std::uint8_t*>(v);
}

// ---- send side ------------------------------------------------------------------------------

// BF16 row to every destination in `mask`; lane d holds the destination row pointer of rank d.
__device__ __forceinline__ void tx_row_bf16(const std::uint8_t* src, std::uint8_t* dst_of_lane, unsigned mask,
                                            int hidden, bool vec_ok) {
    const unsigned lane = ptx::lane_id();
    if (vec_ok) {
        const int chunks = hidden / 8;
        for (int q0 = 0; q0 < chunks; q0 += 128) {
            uint4 v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int q = q0 + u * 32 + lane;
                if (q < chunks) v[u] = ptx::ld_nc_v4(src + static_cast<std::size_t>(q) * 16);
            }
            for (unsigned m = mask; m; m &= m - 1) {
                std::uint8_t* dst = shfl_ptr(dst_of_lane, __ffs(m) - 1);
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int q = q0 + u * 32 + lane;
                    if (q < chunks) ptx::st_v4(dst + static_cast<std::size_t>(q) * 16, v[u]);
                }
            }
        }
    } else {
        const auto* s = reinterpret_cast<const std::uint16_t*>(src);
        for (unsigned m = mask; m; m &= m - 1) {
            auto* dst = reinterpret_cast<std::uint16_t*>(shfl_ptr(dst_of_lane, __ffs(m) - 1));
            for (int i = lane; i < hidden; i += 32) dst[i] = s[i];
        }
    }
}

// FP8 wire: remote destinations get E4M3 bytes, this rank itself keeps the BF16 row.
// Returns the token scale.
__device__ __forceinline__ float tx_row_fp8(const std::uint8_t* src, std::uint8_t* dst_of_lane, unsigned mask,
                                            int self, int hidden, bool vec_ok) {
    const unsigned lane = ptx::lane_id();
    float amax = 0.0f;
    if (vec_ok) {
        const int chunks = hidden / 8;
        for (int q = lane; q < chunks; q += 32) amax = fmaxf(amax, chunk_amax(ptx::ld_nc_v4(src + static_cast<std::size_t>(q) * 16)));
    } else {
        const auto* s = reinterpret_cast<const __nv_bfloat16*>(src);
        for (int i = lane; i < hidden; i += 32) amax = fmaxf(amax, fabsf(__bfloat162float(s[i])));
    }
    amax = warp_max(amax);
    const float scale = fp8_scale_from_amax(amax);
    const float inv = 1.0f / scale;
    if (vec_ok) {
        const int chunks = hidden / 8;
        for (int q0 = 0; q0 < chunks; q0 += 128) {
            uint4 v[4];
            uint2 f[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int q = q0 + u * 32 + lane;
                if (q < chunks) {
                    v[u] = ptx::ld_nc_v4(src + static_cast<std::size_t>(q) * 16);
                    f[u] = chunk_to_fp8(v[u], inv);
                }
            }
            for (unsigned m = mask; m; m &= m - 1) {
                const int d = __ffs(m) - 1;
                std::uint8_t* dst = shfl_ptr(dst_of_lane, d);
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int q = q0 + u * 32 + lane;
                    if (q >= chunks) continue;
                    if (d == self) ptx::st_v4(dst + static_cast<std::size_t>(q) * 16, v[u]);
                    else *reinterpret_cast<uint2*>(dst + static_cast<std::size_t>(q) * 8) = f[u];
                }
            }
        }
    } else {
        const auto* s = reinterpret_cast<const __nv_bfloat16*>(src);
        for (unsigned m = mask; m; m &= m - 1) {
            const int d = __ffs(m) - 1;
            std::uint8_t* dst = shfl_ptr(dst_of_lane, d);
            for (int i = lane; i < hidden; i += 32) {
                if (d == self) reinterpret_cast<__nv_bfloat16*>(dst)[i] = s[i];
                else dst[i] = scalar_to_fp8(s[i], inv);
            }
        }
    }
    return scale;
}

// ---- receive side ----------------------------------------------------------------------------

// One staged row (BF16, or FP8 with `scale`) to `n_rows` output rows; lane i < n_rows holds the
// pointer of output row i in `dst_of_lane`.
__device__ __forceinline__ void rx_row_scatter(const std::uint8_t* src, bool is_fp8, float scale,
                                               std::uint8_t* dst_of_lane, int n_rows, int hidden, bool vec_ok) {
    const unsigned lane = ptx::lane_id();
    if (vec_ok) {
        const int chunks = hidden / 8;
        for (int q0 = 0; q0 < chunks; q0 += 128) {
            uint4 v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int q = q0 + u * 32 + lane;
                if (q < chunks) {
                    if (is_fp8) {
                        uint2 f;
                        asm volatile("ld.global.v2.u32 {%0,%1}, [%2];"
                                     : "=r"(f.x), "=r"(f.y)
                                     : "l"(src + static_cast<std::size_t>(q) * 8)
                                     : "memory");
                        v[u] = chunk_from_fp8(f, scale);
                    } else {
                        v[u] = ptx::ld_v4(src + static_cast<std::size_t>(q) * 16);
                    }
                }
            }
            for (int i = 0; i < n_rows; ++i) {
                std::uint8_t* dst = shfl_ptr(dst_of_lane, i);
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int q = q0 + u * 32 + lane;
                    if (q < chunks) ptx::st_v4(dst + static_cast<std::size_t>(q) * 16, v[u]);
                }
            }
        }
    } else {
        for (int i = 0; i < n_rows; ++i) {
            auto* dst = reinterpret_cast<__nv_bfloat16*>(shfl_ptr(dst_of_lane, i));
            if (is_fp8) {
                const volatile std::uint8_t* s = src;
                for (int k = lane; k < hidden; k += 32) dst[k] = scalar_from_fp8(s[k], scale);
            } else {
                const volatile std::uint16_t* s = reinterpret_cast<const volatile std::uint16_t*>(src);
                for (int k = lane; k < hidden; k += 32) reinterpret_cast<std::uint16_t*>(dst)[k] = s[k];
            }
        }
    }
}

// raw copy of `bytes` (E4M3 codes) from one staged row to n_rows output rows; lane i holds row pointer i
__device__ __forceinline__ void rx_row_copy_bytes(const std::uint8_t* src, std::uint8_t* dst_of_lane, int n_rows, int bytes) {
    const unsigned lane = ptx::lane_id();
    if (bytes % 16 == 0) {
        const int chunks = bytes / 16;
        for (int q0 = 0; q0 < chunks; q0 += 128) {
            uint4 v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int q = q0 + u * 32 + lane;
                if (q < chunks) v[u] = ptx::ld_v4(src + static_cast<std::size_t>(q) * 16);
            }
            for (int i = 0; i < n_rows; ++i) {
                std::uint8_t* dst = shfl_ptr(dst_of_lane, i);
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int q = q0 + u * 32 + lane;
                    if (q < chunks) ptx::st_v4(dst + static_cast<std::size_t>(q) * 16, v[u]);
                }
            }
        }
    } else {
        for (int i = 0; i < n_rows; ++i) {
            std::uint8_t* dst = shfl_ptr(dst_of_lane, i);
            const volatile std::uint8_t* s = src;
            for (int k = lane; k < bytes; k += 32) dst[k] = s[k];
        }
    }
}

__device__ __forceinline__ void zero_row(std::uint8_t* dst, int hidden, bool vec_ok) {
    const unsigned lane = ptx::lane_id();
    if (vec_ok) {
        const uint4 z = make_uint4(0, 0, 0, 0);
        for (int q = lane; q < hidden / 8; q += 32) ptx::st_v4(dst + static_cast<std::size_t>(q) * 16, z);
    } else {
        for (int k = lane; k < hidden; k += 32) reinterpret_cast<std::uint16_t*>(dst)[k] = 0;
    }
}

// bounded wait on a shared-memory mbarrier phase
__device__ __forceinline__ bool mbar_wait_bounded(unsigned long long* bar, unsigned parity, Health& health) {
    while (!ptx::mbar_try_wait(reinterpret_cast<std::uint64_t*>(bar), parity)) {
        if (health.give_up(kErrCopyEngine, static_cast<int>(blockIdx.x), 0)) return false;
    }
    return true;
}

}  // namespace detail


namespace detail {

__device__ __forceinline__ bool warp_failed(const Health& health) {
    return __any_sync(0xffffffffu, health.failed()) != 0;
}
__device__ __forceinline__ bool warp_give_up(Health& health, int code, int context, int detail_value) {
    return __any_sync(0xffffffffu, health.give_up(code, context, detail_value)) != 0;
}

// TMA send of one token: the row is in `slot` (BF16 payload, metadata at meta_off).  Lane d holds the
// destination row of rank d.  Returns false if a copy never completed.
__device__ __forceinline__ void tx_token_tma(const SegmentLayout& lay, unsigned char* slot, std::uint8_t* dst_of_lane,
                                             unsigned mask, int self, bool wire_fp8) {
    // self < 0: no BF16 bypass, this rank's own copy is quantised like everybody else's
    const unsigned lane = ptx::lane_id();
    const unsigned self_bit = self >= 0 ? 1u << self : 0u;
    const unsigned remote = mask & ~self_bit;
    const unsigned bf16_bytes = static_cast<unsigned>(lay.meta_off + lay.meta_bytes);
    const int hidden = lay.hidden;
    if (!wire_fp8 || remote == 0) {
        ptx::fence_proxy_async_smem();
        __syncwarp();
        for (unsigned m = mask; m; m &= m - 1) {
            std::uint8_t* dst = shfl_ptr(dst_of_lane, __ffs(m) - 1);
            if (lane == 0) ptx::bulk_s2g(dst, slot, bf16_bytes);
        }
        if (lane == 0) {
            ptx::bulk_commit();
            ptx::bulk_wait_all();
        }
        __syncwarp();
        return;
    }
    // FP8 wire with at least one remote destination: this rank's own copy leaves first as BF16,
    // then the row is quantised in place and leaves as E4M3 bytes + metadata.
    ptx::fence_proxy_async_smem();
    __syncwarp();
    {
        std::uint8_t* dst = shfl_ptr(dst_of_lane, self >= 0 ? self : 0);
        if ((mask & self_bit) && lane == 0) {
            ptx::bulk_s2g(dst, slot, bf16_bytes);
            ptx::bulk_commit();
            ptx::bulk_wait_read_all();
        }
    }
    __syncwarp();
    const int chunks = hidden / 8;
    float amax = 0.0f;
    for (int q = lane; q < chunks; q += 32) amax = fmaxf(amax, chunk_amax(*reinterpret_cast<const uint4*>(slot + q * 16)));
    amax = warp_max(amax);
    const float scale = fp8_scale_from_amax(amax);
    const float inv = 1.0f / scale;
    // metadata out of the way first (the FP8 layout puts it right behind H bytes)
    uint4 meta_chunk = make_uint4(0, 0, 0, 0);
    const int meta_chunks = lay.meta_bytes / 16;
    if (static_cast<int>(lane) < meta_chunks) meta_chunk = *reinterpret_cast<const uint4*>(slot + lay.meta_off + lane * 16);
    if (lane == 0) meta_chunk.y = __float_as_uint(scale);
    // in-place narrowing, increasing order: chunk q is read before anything lands on it
    for (int q0 = 0; q0 < chunks; q0 += 32) {
        const int q = q0 + lane;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (q < chunks) v = *reinterpret_cast<const uint4*>(slot + q * 16);
        __syncwarp();
        if (q < chunks) *reinterpret_cast<uint2*>(slot + q * 8) = chunk_to_fp8(v, inv);
        __syncwarp();
    }
    if (static_cast<int>(lane) < meta_chunks) *reinterpret_cast<uint4*>(slot + lay.meta_off_fp8 + lane * 16) = meta_chunk;
    ptx::fence_proxy_async_smem();
    __syncwarp();
    const unsigned fp8_bytes = static_cast<unsigned>(lay.meta_off_fp8 + lay.meta_bytes);
    for (unsigned m = remote; m; m &= m - 1) {
        std::uint8_t* dst = shfl_ptr(dst_of_lane, __ffs(m) - 1);
        if (lane == 0) ptx::bulk_s2g(dst, slot, fp8_bytes);
    }
    if (lane == 0) {
        ptx::bulk_commit();
        ptx::bulk_wait_all();
    }
    __syncwarp();
}

}  // namespace detail

__global__ void __launch_bounds__(kMaxWarps * 32, 1) dispatch_kernel(const __grid_constant__ DispatchLaunch launch) {
    using namespace detail;
    const DispatchArgs& a = launch.r[blockIdx.y];
    const RankConst* __restrict__ rc = a.rc;
    const SegmentLayout& lay = rc->lay;

    const int P = lay.num_ranks, C = lay.num_channels, E = lay.num_experts, El = lay.num_local_experts;
    const int K = lay.num_topk, H = lay.hidden, Q = lay.slots, Qf = lay.slots_full;
    const int me = rc->rank, c = blockIdx.x;
    const int T = a.num_tokens;
    const int Tc = (T + C - 1) / C;
    const int t0 = min(T, c * Tc), t1 = min(T, t0 + Tc);
    const int warp = threadIdx.x >> 5;
    const unsigned lane = ptx::lane_id();
    const unsigned lt_mask = (1u << lane) - 1u;
    const unsigned full = 0xffffffffu;
    const int tx_warps = rc->tx_warps, rx_warps = rc->rx_warps;
    const bool vec_ok = rc->vec_ok != 0, use_tma = rc->use_tma != 0, wire_fp8 = rc->wire_fp8 != 0;
    const bool recv_fp8 = rc->recv_fp8 != 0;  // rows stay E4M3 at the receiver (scales in recv_scale); implies wire_fp8
    const int bypass_rank = recv_fp8 ? -1 : me;  // the rank whose own copy stays BF16 under an FP8 wire
    const std::size_t out_row_bytes = static_cast<std::size_t>(H) * (recv_fp8 ? 1 : 2);
    std::uint8_t* const recv_bytes = reinterpret_cast<std::uint8_t*>(a.recv_x);
    const bool ring = rc->ring_mode != 0;
    const int map_stride = 2 + 2 * K;

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
    const int slot_bytes = static_cast<int>(align_up(lay.meta_off + lay.meta_bytes, 128));
    unsigned char* my_slot = smem_raw + slots_at + static_cast<std::size_t>(warp > 0 ? warp - 1 : 0) * slot_bytes;

    Health health(rc, a.error);
    const std::uint64_t epoch = rc->epochs[0] + 1;
    std::uint8_t* my_seg = rc->seg[me];
    std::int64_t* prof = a.profile + static_cast<std::size_t>(c) * 16;
#define BEP_PROF(point) prof[point] = static_cast<std::int64_t>(ptx::globaltimer_ns())

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
        if (use_tma) {
            for (int w = 0; w < kMaxWarps; ++w) ptx::mbar_init(reinterpret_cast<std::uint64_t*>(&sh->mbar[w]), 1);
            ptx::mbar_fence_init();
        }
    }
    const unsigned long long t_start = ptx::globaltimer_ns();
    if (threadIdx.x == 0) {
        prof[kProfStart] = static_cast<std::int64_t>(t_start);
        prof[kProfFirstRxRow] = 0;
        prof[kProfFirstTxDone] = 0;
    }

    // Reuse guard: nothing of this epoch may reach a peer before that peer has finished reading the
    // previous epoch out of its segment (reference: the counts_consumed == epoch-1 wait of
    // advanced_begin_epoch, advanced_layout.cuh:9-89).  The flags are local; the wait is normally free.
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
    // (reference: advanced_route_flags + advanced_stable_ordinals + advanced_prepare_channels_parallel,
    //  advanced_layout.cuh:287-425; here O(T*K) with one barrier instead of O((P+E)*T) block scans)
    if (!a.cached) {
        for (int i = threadIdx.x; i < E; i += blockDim.x) {
            cnt_e[i] = 0;
            bits_e[i] = 0;
        }
        if (threadIdx.x < kMaxRanks) {
            sh->cnt_r[threadIdx.x] = 0;
            sh->bits_r[threadIdx.x] = 0;
        }
        __syncthreads();
        for (int t = t0 + threadIdx.x; t < t1; t += blockDim.x) {
            unsigned mask = 0;
            const std::int64_t* row = a.topk_idx + static_cast<std::size_t>(t) * K;
            for (int k = 0; k < K; ++k) {
                const std::int64_t e = row[k];
                if (e == -1) continue;
                bool bad = e < -1 || e >= E;
                for (int k2 = 0; k2 < k && !bad; ++k2) bad = row[k2] == e;
                if (bad) {
                    record_error(rc, a.error, kErrInvalidRouting, t, k);
                    continue;
                }
                mask |= 1u << static_cast<int>(e / El);
                atomicAdd(&cnt_e[e], 1);
            }
            a.plan_mask[t] = mask;
            for (unsigned m = mask; m; m &= m - 1) atomicAdd(&sh->cnt_r[__ffs(m) - 1], 1);
        }
        __syncthreads();
        int* hist = rc->block_hist + static_cast<std::size_t>(c) * (E + P);
        for (int i = threadIdx.x; i < E + P; i += blockDim.x) hist[i] = i < E ? cnt_e[i] : sh->cnt_r[i - E];
        if (threadIdx.x == 0) BEP_PROF(kProfHistDone);
        grid_barrier(&rc->grid_bar[0], health);
        if (threadIdx.x == 0) BEP_PROF(kProfBarrierDone);
        // exclusive prefix over earlier channels (stable order = channel order = token order)
        for (int i = threadIdx.x; i < E + P; i += blockDim.x) {
            int base = 0, total = 0;
            for (int c2 = 0; c2 < C; ++c2) {
                const int v = __ldcg(rc->block_hist + static_cast<std::size_t>(c2) * (E + P) + i);
                total += v;
                if (c2 < c) base += v;
            }
            if (i < E) {
                cnt_e[i] = base;
                total_e[i] = total;
            } else {
                sh->cnt_r[i - E] = 0;  // row indices at a destination are channel-relative
                sh->total_r[i - E] = total;
            }
        }
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
    // expect (counts message; reference: publish_counts, layout.cuh:7-29 -- channel d, d+C, ... serves
    // destination d), warp 0 numbers this channel's tokens.
    if (warp == 1 && !rc->test_withhold_counts) {
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
    if (!a.cached) {
    if (warp == 0) {
        // Stable ordinals, 32 tokens at a time: lane = token.  bits_*[bin] collects which lanes hit a
        // bin; an ordinal is (tokens before this chunk) + (lower lanes in the bin).
        for (int base_t = t0; base_t < t1; base_t += 32) {
            const int t = base_t + lane;
            const bool active = t < t1;
            const unsigned mask = active ? a.plan_mask[t] : 0u;
            const std::int64_t* row = a.topk_idx + static_cast<std::size_t>(active ? t : 0) * K;
            for (int k = 0; k < K; ++k) {
                const std::int64_t e = active ? row[k] : -1;
                if (e >= 0 && e < E) atomicOr(&bits_e[e], 1u << lane);
            }
            for (unsigned m = mask; m; m &= m - 1) atomicOr(&sh->bits_r[__ffs(m) - 1], 1u << lane);
            __syncwarp();
            if (active) {
                for (int k = 0; k < K; ++k) {
                    const std::int64_t e = row[k];
                    a.plan_expert_ord[static_cast<std::size_t>(t) * K + k] =
                        (e >= 0 && e < E) ? cnt_e[e] + __popc(bits_e[e] & lt_mask) : -1;
                }
                for (int d = 0; d < P; ++d)
                    a.plan_slot[static_cast<std::size_t>(t) * P + d] =
                        (mask >> d & 1u) ? sh->cnt_r[d] + __popc(sh->bits_r[d] & lt_mask) : -1;
            }
            __syncwarp();
            for (int k = 0; k < K; ++k) {
                const std::int64_t e = active ? row[k] : -1;
                if (e >= 0 && e < E) {
                    const unsigned b = bits_e[e];
                    if (lane == 31u - __clz(b)) cnt_e[e] += __popc(b);
                }
            }
            for (unsigned m = mask; m; m &= m - 1) {
                const int d = __ffs(m) - 1;
                const unsigned b = sh->bits_r[d];
                if (lane == 31u - __clz(b)) sh->cnt_r[d] += __popc(b);
            }
            __syncwarp();
            for (int k = 0; k < K; ++k) {
                const std::int64_t e = active ? row[k] : -1;
                if (e >= 0 && e < E) bits_e[e] = 0;
            }
            for (unsigned m = mask; m; m &= m - 1) sh->bits_r[__ffs(m) - 1] = 0;
            __syncwarp();
        }
    }
        if (warp == 0 && lane == 0) BEP_PROF(kProfOrdinalsDone);
    }
    if (cta_failed(health, &sh->cta_flag)) return;
    if (threadIdx.x == 0) BEP_PROF(kProfRolesSplit);

    // ---- role split ------------------------------------------------------------------------------
    unsigned long long st_source = 0, st_remote_rows = 0, st_deliveries = 0, st_early = 0, st_probes = 0,
                       st_credit = 0, st_local = 0, st_published = 0;

    if (warp == 0) {
        // ===== control: receive prefix (reference: advanced_prepare_receive_prefixes,
        // advanced_layout.cuh:94-195), then zero padding =====
        const unsigned long long prefix_t0 = ptx::globaltimer_ns();
        if (lane < static_cast<unsigned>(P)) {
            const std::uint64_t* flag = flag_ptr(my_seg, lay.counts_flag_off, lane);
            while (ptx::ld_acquire_sys(flag) != epoch) {
                if (health.give_up(kErrCountsWait, lane, 0)) break;
            }
        }
        __syncwarp();
        if (lane == 0) BEP_PROF(kProfCountsArrived);
        test_delay(rc->delay_prefix_ns);
        const bool bad = warp_failed(health);
        if (!bad) {
            const int stride = lay.counts_stride;
            {   // bring all P messages into shared memory with wide, independent loads
                const uint4* g = reinterpret_cast<const uint4*>(my_seg + lay.counts_off);
                uint4* d4 = reinterpret_cast<uint4*>(msg_sm);
                for (int i = lane; i < P * stride / 4; i += 32) d4[i] = ptx::ld_v4(g + i);
            }
            __syncwarp();
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
            if (carry > rc->expanded_cap || unique_total > rc->unique_cap) {
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
                BEP_PROF(kProfPrefixReady);
            }
            // zero padding between expert segments (reference: advanced_zero_padding,
            // advanced_layout.cuh:250-265): channel c takes local experts c, c+C, ...
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
        }
    } else if (warp <= tx_warps) {
        // ===== send =====
        const int w = warp - 1;
        unsigned parity = 0;
        unsigned char* meta_sm = use_tma ? my_slot + lay.meta_off : sh->meta[warp];
        const unsigned self_bit = 1u << me;
        const bool delayed = (w == tx_warps - 1);
        for (int i = w; t0 + i < t1; i += tx_warps) {
            if (warp_failed(health)) break;
            const int t = t0 + i;
            const unsigned mask = a.plan_mask[t];
            if (mask == 0) continue;
            // destination row of lane d; ring mode first waits for the slot's credit
            int j = -1;
            std::uint8_t* dst = nullptr;
            std::uint64_t* ready = nullptr;
            if (lane < static_cast<unsigned>(P) && (mask >> lane & 1u)) {
                j = a.plan_slot[static_cast<std::size_t>(t) * P + lane];
                const std::size_t ring_index = (static_cast<std::size_t>(me) * C + c) * Q + (j % Q);
                dst = rc->seg[lane] + lay.stage_off + ring_index * lay.row_stride;
                ready = reinterpret_cast<std::uint64_t*>(rc->seg[lane] + lay.ready_off) + ring_index;
                if (ring && j >= Q) {
                    const std::uint64_t* ack = reinterpret_cast<const std::uint64_t*>(my_seg + lay.ack_off) +
                                               (static_cast<std::size_t>(lane) * C + c) * Q + (j % Q);
                    const std::uint64_t want = make_seq(epoch, static_cast<std::uint32_t>(j - Q + 1));
                    bool missed = false;
                    while (ptx::ld_acquire_sys(ack) != want) {
                        missed = true;
                        if (health.give_up(kErrCreditWait, lane, j)) break;
                    }
                    if (missed) ++st_credit;
                }
            }
            __syncwarp();
            if (warp_failed(health)) break;
            const std::uint8_t* src = reinterpret_cast<const std::uint8_t*>(a.x + static_cast<std::size_t>(t) * H);
            std::uint64_t* bar = reinterpret_cast<std::uint64_t*>(&sh->mbar[warp]);
            if (use_tma && lane == 0) {
                ptx::mbar_expect_tx(bar, static_cast<unsigned>(H) * 2);
                ptx::bulk_g2s(my_slot, src, static_cast<unsigned>(H) * 2, bar);
            }
            // metadata: header | expert[K] | ordinal[K] | weight[K]
            if (delayed) test_delay(rc->delay_meta_ns);
            if (lane == 0) {
                reinterpret_cast<int*>(meta_sm)[0] = t;
                reinterpret_cast<float*>(meta_sm)[1] = 1.0f;
                reinterpret_cast<int*>(meta_sm)[2] = 0;
                reinterpret_cast<int*>(meta_sm)[3] = 0;
            }
            for (int k = lane; k < K; k += 32) {
                const std::int64_t e = a.topk_idx[static_cast<std::size_t>(t) * K + k];
                reinterpret_cast<int*>(meta_sm + 16)[k] = (e >= 0 && e < E) ? static_cast<int>(e) : -1;
                reinterpret_cast<int*>(meta_sm + 16)[K + k] = a.plan_expert_ord[static_cast<std::size_t>(t) * K + k];
                reinterpret_cast<float*>(meta_sm + 16)[2 * K + k] =
                    a.topk_w ? a.topk_w[static_cast<std::size_t>(t) * K + k] : 1.0f;
            }
            for (int b = 16 + 12 * K + lane; b < lay.meta_bytes; b += 32) meta_sm[b] = 0;
            __syncwarp();
            if (lane == 0 && sh->first_tx_ns == 0) atomicCAS(&sh->first_tx_ns, 0ull, ptx::globaltimer_ns());
            if (delayed) test_delay(rc->delay_tx_ns);
            if (!use_tma) {
                float scale = 1.0f;
                if (wire_fp8 && (recv_fp8 || (mask & ~self_bit))) scale = tx_row_fp8(src, dst, mask, bypass_rank, H, vec_ok);
                else tx_row_bf16(src, dst, mask, H, vec_ok);
                if (lane == 0) reinterpret_cast<float*>(meta_sm)[1] = scale;
                __syncwarp();
                for (unsigned m = mask; m; m &= m - 1) {
                    const int d = __ffs(m) - 1;
                    std::uint8_t* row = shfl_ptr(dst, d);
                    std::uint8_t* mdst = row + ((wire_fp8 && d != bypass_rank) ? lay.meta_off_fp8 : lay.meta_off);
                    for (int q = lane; q < lay.meta_bytes / 16; q += 32)
                        ptx::st_v4(mdst + q * 16, *reinterpret_cast<const uint4*>(meta_sm + q * 16));
                }
            } else {
                const bool arrived = mbar_wait_bounded(&sh->mbar[warp], parity, health);
                parity ^= 1u;
                if (!__all_sync(full, arrived)) break;
                tx_token_tma(lay, my_slot, dst, mask, bypass_rank, wire_fp8);
            }
            __syncwarp();
            // publish: READY of this row at every destination (one lane per destination releases)
            if (j >= 0) ptx::st_release_sys(ready, make_seq(epoch, static_cast<std::uint32_t>(j + 1)));
            if (lane == 0) {
                if (mask & ~self_bit) {
                    ++st_source;
                    st_deliveries += __popc(mask & ~self_bit);
                }
                if (mask & self_bit) ++st_local;
                st_published += __popc(mask);
                if (*reinterpret_cast<volatile int*>(&sh->prefix_ready) == 0) ++st_early;
                if (w == 0 && st_published == static_cast<unsigned long long>(__popc(mask))) BEP_PROF(kProfFirstTxDone);
            }
        }
        if (lane == 0) atomicMax(&sh->last_tx_ns, ptx::globaltimer_ns());
        if (w == 0 && lane == 0) BEP_PROF(kProfTxDone);
    } else {
        // ===== receive + expand =====
        const int w = warp - 1 - tx_warps;
        const bool delayed = (w == rx_warps - 1);
        // The control warp owns the diagnosis of a missing counts message (it knows which source is
        // late); this wait only has to end, so its own deadline is a quarter of the timeout later.
        health.deadline += rc->timeout_ns / 4;
        while (*reinterpret_cast<volatile int*>(&sh->prefix_ready) == 0) {
            if (warp_give_up(health, kErrCountsWait, -1, 0)) break;
        }
        __threadfence_block();
        __syncwarp();
        if (!warp_failed(health) && *reinterpret_cast<volatile int*>(&sh->prefix_ready) != 0) {
            int next_j = w;
            const int expect = lane < static_cast<unsigned>(P) ? sh->chan_expected[lane] : 0;
            const std::uint64_t* ready_base = reinterpret_cast<const std::uint64_t*>(my_seg + lay.ready_off);
            unsigned parity = 0;
            std::uint64_t* bar = reinterpret_cast<std::uint64_t*>(&sh->mbar[warp]);
            while (true) {
                const bool pending = lane < static_cast<unsigned>(P) && next_j < expect;
                const unsigned pend = __ballot_sync(full, pending);
                if (pend == 0) break;
                bool hit = false;
                if (pending) {
                    const std::uint64_t v =
                        ptx::ld_acquire_sys(ready_base + (static_cast<std::size_t>(lane) * C + c) * Q + (next_j % Q));
                    hit = v == make_seq(epoch, static_cast<std::uint32_t>(next_j + 1));
                }
                const unsigned hits = __ballot_sync(full, hit);
                if (hits == 0) {
                    ++st_probes;
                    if (warp_give_up(health, kErrRowWait, __ffs(pend) - 1, 0)) break;
                    continue;
                }
                bool stop = false;
                for (unsigned hm = hits; hm && !stop; hm &= hm - 1) {
                    const int s = __ffs(hm) - 1;
                    const int j = __shfl_sync(full, next_j, s);
                    if (lane == static_cast<unsigned>(s)) next_j += rx_warps;
                    const bool fp8row = wire_fp8 && s != bypass_rank;
                    const std::size_t ring_index = (static_cast<std::size_t>(s) * C + c) * Q + (j % Q);
                    const std::uint8_t* row_src = my_seg + lay.stage_off + ring_index * lay.row_stride;
                    const int moff = fp8row ? lay.meta_off_fp8 : lay.meta_off;
                    if (delayed) test_delay(rc->delay_rx_ns);
                    const unsigned char* meta;
                    if (use_tma) {
                        ptx::fence_proxy_async();
                        if (lane == 0) {
                            const unsigned bytes = static_cast<unsigned>(moff + lay.meta_bytes);
                            ptx::bulk_wait_read_all();  // the previous row's stores have left the buffer
                            ptx::mbar_expect_tx(bar, bytes);
                            ptx::bulk_g2s(my_slot, row_src, bytes, bar);
                        }
                        const bool arrived = mbar_wait_bounded(&sh->mbar[warp], parity, health);
                        parity ^= 1u;
                        if (!__all_sync(full, arrived)) {
                            stop = true;
                            break;
                        }
                        meta = my_slot + moff;
                    } else {
                        meta = row_src + moff;
                    }
                    // metadata -> registers
                    int token;
                    float scale;
                    if (use_tma) {
                        token = reinterpret_cast<const int*>(meta)[0];
                        scale = reinterpret_cast<const float*>(meta)[1];
                    } else {
                        token = ptx::ld_volatile(reinterpret_cast<const int*>(meta));
                        scale = __int_as_float(ptx::ld_volatile(reinterpret_cast<const int*>(meta) + 1));
                    }
                    int e = -1, ord = 0;
                    float wgt = 0.0f;
                    if (lane < static_cast<unsigned>(K)) {
                        const int* mi = reinterpret_cast<const int*>(meta + 16);
                        if (use_tma) {
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
                    const bool local = e >= 0 && e / El == me;
                    const int el = local ? e - me * El : -1;
                    const unsigned lmask = __ballot_sync(full, local);
                    const int n_local = __popc(lmask);
                    const int pos = __popc(lmask & lt_mask);
                    int* map = a.comb_map + ((static_cast<std::size_t>(s) * C + c) * Qf + j) * map_stride;
                    // output rows: lane i < n_rows holds row pointer i
                    std::uint8_t* out_ptr = nullptr;
                    int n_rows;
                    bool overflow = false;
                    if (a.do_expand) {
                        n_rows = n_local;
                        int row = -1;
                        if (local) {
                            row = eoff[el] + spre[s * El + el] + ord;
                            overflow = row < 0 || row >= rc->expanded_cap;
                        }
                        // compact: the i-th local slot's row goes to lane i
                        for (unsigned lm = lmask, i = 0; lm; lm &= lm - 1, ++i) {
                            const int r = __shfl_sync(full, row, __ffs(lm) - 1);
                            if (lane == i) out_ptr = recv_bytes + static_cast<std::size_t>(r) * out_row_bytes;
                        }
                        if (local && !overflow) {
                            if (recv_fp8) a.recv_scale[row] = scale;
                            a.recv_idx[row] = el;
                            a.recv_w[row] = wgt;
                            a.source_meta[static_cast<std::size_t>(row) * 3 + 0] = s;
                            a.source_meta[static_cast<std::size_t>(row) * 3 + 1] = token;
                            a.source_meta[static_cast<std::size_t>(row) * 3 + 2] = lane;
                            map[2 + 2 * pos] = row;
                            map[3 + 2 * pos] = __float_as_int(wgt);
                        }
                    } else {
                        n_rows = 1;
                        const int row = sh->source_offsets[s] + sh->chan_base[s] + j;
                        overflow = row >= rc->unique_cap;
                        if (lane == 0) out_ptr = recv_bytes + static_cast<std::size_t>(row) * out_row_bytes;
                        if (!overflow) {
                            if (recv_fp8 && lane == 0) a.recv_scale[row] = scale;
                            if (lane < static_cast<unsigned>(K)) {
                                a.recv_idx[static_cast<std::size_t>(row) * K + lane] = el;
                                a.recv_w[static_cast<std::size_t>(row) * K + lane] = local ? wgt : 0.0f;
                            }
                            if (lane == 0) {
                                a.source_meta[static_cast<std::size_t>(row) * 3 + 0] = s;
                                a.source_meta[static_cast<std::size_t>(row) * 3 + 1] = token;
                                a.source_meta[static_cast<std::size_t>(row) * 3 + 2] = -1;
                                map[2] = row;
                                map[3] = __float_as_int(1.0f);
                            }
                        }
                    }
                    if (lane == 0) {
                        map[0] = token;
                        map[1] = a.do_expand ? n_local : 1;
                    }
                    if (__any_sync(full, overflow)) {
                        if (lane == 0) record_error(rc, a.error, kErrCapacity, s, j);
                        stop = true;
                        break;
                    }
                    if (delayed) test_delay(rc->delay_scatter_ns);
                    std::uint64_t* ack = reinterpret_cast<std::uint64_t*>(rc->seg[s] + lay.ack_off) +
                                         (static_cast<std::size_t>(me) * C + c) * Q + (j % Q);
                    if (!use_tma) {
                        if (recv_fp8) rx_row_copy_bytes(row_src, out_ptr, n_rows, H);
                        else rx_row_scatter(row_src, fp8row, scale, out_ptr, n_rows, H, vec_ok);
                        if (ring) {
                            __syncwarp();
                            if (lane == 0) ptx::st_release_sys(ack, make_seq(epoch, static_cast<std::uint32_t>(j + 1)));
                        }
                    } else {
                        // the row is in shared memory: its ring slot can be handed back already
                        if (ring && lane == 0) ptx::st_release_sys(ack, make_seq(epoch, static_cast<std::uint32_t>(j + 1)));
                        if (fp8row && !recv_fp8) {
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
                        }
                        for (int i = 0; i < n_rows; ++i) {
                            std::uint8_t* dst = shfl_ptr(out_ptr, i);
                            if (lane == 0) ptx::bulk_s2g(dst, my_slot, static_cast<unsigned>(out_row_bytes));
                        }
                        if (lane == 0) ptx::bulk_commit();
                    }
                    if (lane == 0 && s != me) ++st_remote_rows;
                    if (w == 0 && lane == 0 && prof[kProfFirstRxRow] == 0) BEP_PROF(kProfFirstRxRow);
                }
                if (stop) break;
            }
            if (w == 0 && lane == 0) BEP_PROF(kProfRxDone);
        }
    }

    // ---- epilogue ----------------------------------------------------------------------------------
    __syncwarp();
    if (lane == 0) {
        if (use_tma) ptx::bulk_wait_all();
        atomicAdd(&sh->stat[kStatSourceTokens], st_source);
        atomicAdd(&sh->stat[kStatRemoteRows], st_remote_rows);
        atomicAdd(&sh->stat[kStatDeliveries], st_deliveries);
        atomicAdd(&sh->stat[kStatEarlyRows], st_early);
        atomicAdd(&sh->stat[kStatRxEmptyProbes], st_probes);
        atomicAdd(&sh->stat[kStatCreditMisses], st_credit);
        atomicAdd(&sh->stat[kStatLocalRows], st_local);
        atomicAdd(&sh->stat[kStatRowsPublished], st_published);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned long long t_end = ptx::globaltimer_ns();
        prof[kProfEnd] = static_cast<std::int64_t>(t_end);
        std::int64_t* cs = rc->chan_stats + static_cast<std::size_t>(c) * 10;
        for (int i = 0; i < 8; ++i) cs[i] = static_cast<std::int64_t>(sh->stat[i]);
        cs[8] = static_cast<std::int64_t>(t_start);
        cs[9] = static_cast<std::int64_t>(t_end);
        a.prefix_tx_ts[(c + 1) * 2 + 0] = static_cast<std::int64_t>(sh->first_tx_ns);
        a.prefix_tx_ts[(c + 1) * 2 + 1] = static_cast<std::int64_t>(sh->last_tx_ns);
        __threadfence();
        const unsigned long long old = atomicAdd(&rc->done_ctas[0], 1ull);
        if ((old + 1) % static_cast<unsigned long long>(C) == 0) {
            // last channel of this rank: statistics (reference: advanced_reduce_statistics,
            // advanced_layout.cuh:267-283), hand the staging area back to every source, advance the epoch
            __threadfence();
            std::int64_t sum[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            std::int64_t first = INT64_MAX, last = 0;
            for (int c2 = 0; c2 < C; ++c2) {
                const std::int64_t* o = rc->chan_stats + static_cast<std::size_t>(c2) * 10;
                for (int i = 0; i < 8; ++i) sum[i] += __ldcg(o + i);
                first = min(first, __ldcg(o + 8));
                last = max(last, __ldcg(o + 9));
            }
            for (int i = 0; i < 8; ++i) a.stats[i] = sum[i];
            a.timestamps[0] = first;
            a.timestamps[1] = last;
            if (!health.failed()) {
                for (int p = 0; p < P; ++p)
                    if (p != rc->test_skip_done_to) ptx::st_release_sys(flag_ptr(rc->seg[p], lay.done_off, me), epoch);
            }
            rc->epochs[0] = epoch;
        }
    }
}

#endif  // __CUDACC__

}  // namespace bep
