// What the roles of the dispatch kernel share: the per-CTA context and shared-memory layout, the opt-in role
// instrumentation, and the row-level helpers (copies through registers, FP8 quantisation of a row in shared memory,
// row metadata, bounded mbarrier waits, placement of a received row into its output rows).
#pragma once

#include "protocol.cuh"
#include "quant.cuh"

#ifndef BEP_ENABLE_PROFILING
#define BEP_ENABLE_PROFILING 0
#endif

namespace bep {

constexpr int kMetaSmemBytes = 16 + 12 * kMaxTopk;
constexpr int kFlagLag = 2;         // a row's READY flags are released after at least this many later rows were issued
constexpr int kFlagBatch = 8;       // READY flags of up to this many rows share one system-scope fence

struct DispatchShared;

// What the roles of one CTA work from.  It lives in shared memory (DispatchShared::ctx), written once before the roles
// split: as a local variable of the kernel it sat in local memory, and the roles' loads of its fields missed L1 four
// times out of ten (measured), each a round trip to L2 in the middle of a row.
struct Ctx {
    const DispatchArgs* a;
    const RankConst* rc;
    DispatchShared* sh;
    int* eoff;                   // [El+1] aligned offsets of the local experts (valid once prefix_ready)
    int* spre;                   // [P][El] rows of earlier sources inside each expert segment
    unsigned char* row_buffers;  // bulk-copy engine: first row buffer
    int* send_tiles;             // bulk-copy engine: one metadata tile [32][P + 3K] per send warp
    std::uint8_t* my_seg;
    std::uint8_t* recv_bytes;
    std::int64_t* prof;
    std::int64_t* role_prof;     // [warps][kRoleFields] of this channel (profiling builds), else nullptr
    std::size_t out_row_bytes;
    std::uint64_t epoch;
    int slot_bytes, stages;
    int P, C, E, El, K, H, Q, Qf, me, c, t0, t1, rx_warps, map_stride;
    int T, Tc;                         // tokens of this rank, tokens per channel
    int send_warps;                    // send warps in this CTA
    int send_first, send_stride;       // channels this CTA's send warps serve: send_first, send_first + send_stride, ... < C
    int rx_buffer_base;                // index of the first receive warp's row buffer
    bool vec_ok, use_tma, wire_fp8, recv_fp8, ring;
    bool plan_is_foreign;              // the send warps read a plan that other CTAs write during this launch
    bool fence_flags, fence_every_lane, corrupt_sequence;
    // copies of what the roles read per row from the rank's constants (those live in global memory)
    int expanded_cap, unique_cap;
    std::uint64_t delay_meta_ns, delay_tx_ns, delay_rx_ns, delay_scatter_ns, timeout_ns;
    std::uint8_t* seg[kMaxRanks];
    SegmentLayout lay;
};

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
    unsigned long long mbar[kMaxRowBuffers];
    unsigned long long prefix_bar;  // the control warp arrives once the receive prefix is settled (prefix_ready says how)
    Ctx ctx;
    alignas(16) unsigned char meta[kMaxWarps][kMetaSmemBytes];
};

// Dynamic shared memory: header | cnt_e[E] | bits_e[E] | total_e[E] | eoff[El+1] | ecount[El] |
// spre[P*El] | msg[P*counts_stride] | (bulk-copy engine only) `stages` row buffers per send warp and one
// per receive warp.
inline std::size_t dispatch_smem_bytes(const SegmentLayout& lay, int tx_warps, int rx_warps, bool use_tma, int stages,
                                       int send_ctas) {
    std::size_t bytes = align_up(sizeof(DispatchShared), 16);
    bytes += static_cast<std::size_t>(lay.num_experts) * 12;
    bytes += static_cast<std::size_t>(lay.num_local_experts) * 8 + 4;
    bytes += static_cast<std::size_t>(lay.num_ranks) * lay.num_local_experts * 4;
    bytes = align_up(bytes, 16) + static_cast<std::size_t>(lay.num_ranks) * lay.counts_stride * 4;
    bytes = align_up(bytes, 128);
    if (use_tma) {
        bytes += static_cast<std::size_t>(dispatch_row_buffer_count(tx_warps, rx_warps, stages, send_ctas)) *
                 align_up(lay.meta_off + lay.meta_bytes, 128);
        bytes += static_cast<std::size_t>(tx_warps) * 32 * (lay.num_ranks + 3 * lay.num_topk) * 4;  // send warps' metadata tiles
    }
    return bytes;
}

#ifdef __CUDACC__

// ---- opt-in role instrumentation ---------------------------------------------------------------
// Built only with -DBEP_ENABLE_PROFILING=1 (a separate library): every send and receive warp adds up, in
// registers, how long it spent in each kind of wait and how many rows it handled, and lane 0 writes the
// sixteen counters of its warp once, when the role ends.  A normal build contains none of this.
enum RoleField : int {
    kRoleRows = 0,         // rows sent (send warps) / delivered (receive warps)
    kRoleTotalNs = 1,      // role start to role end
    kRoleLoadWaitNs = 2,   // waiting for a row to land in shared memory (mbarrier)
    kRoleStoreWaitNs = 3,  // send: waiting for a bulk group to complete before its flags / receive: for a buffer to drain
    kRoleCreditWaitNs = 4, // send, ring mode: waiting for slot credit
    kRolePrefixWaitNs = 5, // receive: waiting for the receive prefix
    kRoleIdlePollNs = 6,   // receive: probes that found no row
    kRoleMetaNs = 7,       // building (send) or decoding and placing (receive) row metadata
    kRoleLocalRows = 8,    // receive: rows taken straight from x
    kRoleQuantNs = 9,      // FP8 conversion in shared memory
    kRoleIssueNs = 10,     // issuing the outgoing copies
    kRoleBufferWaitNs = 11, // send: waiting for a row buffer's previous row to have left it before it is refilled
    kRoleFirstBatchNs = 12, // send: role start until the first batch of routing metadata is in shared memory
    kRoleFirstIssueNs = 13, // send: role start until the first row's copies have been issued
    kRoleDrainNs = 14,      // send: the final wait for the last rows' copies, up to their flags
    kRoleFields = kRoleFieldCount,
};
#if BEP_ENABLE_PROFILING
#define BEP_ROLE_DECL() unsigned long long role_prof[kRoleFields] = {0}; const unsigned long long role_t_begin = ptx::globaltimer_ns()
#define BEP_ROLE_T(var) const unsigned long long var = ptx::globaltimer_ns()
#define BEP_ROLE_ADD(field, since) role_prof[field] += ptx::globaltimer_ns() - (since)
#define BEP_ROLE_COUNT(field, n) role_prof[field] += (n)
#define BEP_ROLE_MARK(field) do { if (role_prof[field] == 0) role_prof[field] = ptx::globaltimer_ns() - role_t_begin; } while (0)
#define BEP_ROLE_FLUSH(dst)                                                                        \
    do {                                                                                           \
        role_prof[kRoleTotalNs] = ptx::globaltimer_ns() - role_t_begin;                            \
        if (ptx::lane_id() == 0 && (dst) != nullptr)                                               \
            for (int f_ = 0; f_ < kRoleFields; ++f_) (dst)[f_] = static_cast<std::int64_t>(role_prof[f_]); \
    } while (0)
#else
#define BEP_ROLE_DECL() do {} while (0)
#define BEP_ROLE_T(var) do {} while (0)
#define BEP_ROLE_ADD(field, since) do {} while (0)
#define BEP_ROLE_COUNT(field, n) do {} while (0)
#define BEP_ROLE_MARK(field) do {} while (0)
#define BEP_ROLE_FLUSH(dst) do {} while (0)
#endif

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

// FP8: every destination gets E4M3 bytes except lane `self` (pass -1 for none), which keeps BF16.
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

// all but the N most recent bulk groups of this thread are complete (their global writes performed)
template <int N>
__device__ __forceinline__ void bulk_wait_group() {
    asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}
// all but the N most recent bulk groups of this thread have finished reading shared memory
template <int N>
__device__ __forceinline__ void bulk_wait_group_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}

// Values every role of one channel CTA needs; filled once by the kernel.

struct RoleStats {
    unsigned long long source = 0, remote_rows = 0, deliveries = 0, early = 0, probes = 0, credit = 0, local = 0,
                       published = 0;
};

// What a send warp keeps in registers for one token: lane d holds the row index at destination d,
// lane k the k-th expert id, its ordinal and its weight.
struct TokenRegs {
    int t;
    int ch;         // the token's channel
    unsigned mask;  // remote destinations only
    int j;
    int e, ord;
    float w;
};

// Row metadata behind the payload: {src_token, scale, seq_epoch, seq_index} | expert[K] | ordinal[K] | weight[K].
// The sequence words let the receiver check that the payload it reads belongs to this epoch and to the token the
// header names: a READY flag that overtook its payload would expose the previous epoch's row.
__device__ __forceinline__ void write_row_meta(unsigned char* meta, const SegmentLayout& lay, int token, float scale,
                                               std::uint32_t seq_epoch, int e, int ord, float w, int K) {
    const unsigned lane = ptx::lane_id();
    if (lane == 0) {
        reinterpret_cast<int*>(meta)[0] = token;
        reinterpret_cast<float*>(meta)[1] = scale;
        reinterpret_cast<std::uint32_t*>(meta)[2] = seq_epoch;
        reinterpret_cast<std::uint32_t*>(meta)[3] = static_cast<std::uint32_t>(token) + 1u;
    }
    if (lane < static_cast<unsigned>(K)) {
        reinterpret_cast<int*>(meta + 16)[lane] = e;
        reinterpret_cast<int*>(meta + 16)[K + lane] = ord;
        reinterpret_cast<float*>(meta + 16)[2 * K + lane] = w;
    }
    for (int b = 16 + 12 * K + lane; b < lay.meta_bytes; b += 32) meta[b] = 0;
}

// Up to eight expert ids of one token into registers: 16-byte read-only loads when the row allows them (the ids are
// an input of the launch, nothing writes them).  Entries past `left` read as -1.
__device__ __forceinline__ void load_experts8(const std::int64_t* p, int left, std::int64_t (&e)[8]) {
    if (left >= 8 && (reinterpret_cast<std::uintptr_t>(p) & 15u) == 0) {
        const longlong2* p2 = reinterpret_cast<const longlong2*>(p);
        longlong2 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) v[u] = __ldg(p2 + u);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            e[2 * u] = v[u].x;
            e[2 * u + 1] = v[u].y;
        }
    } else {
#pragma unroll
        for (int u = 0; u < 8; ++u) e[u] = u < left ? __ldg(p + u) : -1;
    }
}

__device__ __forceinline__ void load_token_routes(const DispatchArgs& a, int t, int K, int E, int& e, int& ord, float& w) {
    const unsigned lane = ptx::lane_id();
    e = -1;
    ord = -1;
    w = 0.0f;
    if (lane < static_cast<unsigned>(K)) {
        const std::int64_t e64 = a.topk_idx[static_cast<std::size_t>(t) * K + lane];
        e = (e64 >= 0 && e64 < E) ? static_cast<int>(e64) : -1;
        ord = a.plan_expert_ord[static_cast<std::size_t>(t) * K + lane];
        w = a.topk_w ? a.topk_w[static_cast<std::size_t>(t) * K + lane] : 1.0f;
    }
}

// BF16 row in shared memory -> E4M3 codes in its first half; returns the row scale.  Four 16-byte chunks per lane and
// step (128 chunks per step): the codes of a step land on bytes [8 q0, 8 q0 + 1024), that is on input chunks
// [q0 / 2, q0 / 2 + 64).  Only in the first step do these overlap the chunks the step itself reads, and there every
// lane has read before any lane writes (the barrier); from the second step on they lie wholly below q0, in chunks
// consumed by earlier steps, and the chunks of later steps start above every byte written so far.  So one barrier per
// step is enough.  With dedicated sender CTAs a few warps quantise every row of the rank, and this loop is their
// critical path: at hidden 7168 it went from 56 barrier-separated steps of one chunk per lane to 7 + 7 steps.
__device__ __forceinline__ float quantise_row_in_place(unsigned char* slot, int hidden) {
    const unsigned lane = ptx::lane_id();
    const int chunks = hidden / 8;
    float amax = 0.0f;
    for (int q0 = 0; q0 < chunks; q0 += 128) {
        uint4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int q = q0 + u * 32 + static_cast<int>(lane);
            v[u] = q < chunks ? *reinterpret_cast<const uint4*>(slot + q * 16) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) amax = fmaxf(amax, chunk_amax(v[u]));
    }
    amax = warp_max(amax);
    const float scale = fp8_scale_from_amax(amax);
    const float inv = 1.0f / scale;
    for (int q0 = 0; q0 < chunks; q0 += 128) {
        uint4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int q = q0 + u * 32 + static_cast<int>(lane);
            v[u] = q < chunks ? *reinterpret_cast<const uint4*>(slot + q * 16) : make_uint4(0, 0, 0, 0);
        }
        __syncwarp();
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int q = q0 + u * 32 + static_cast<int>(lane);
            if (q < chunks) *reinterpret_cast<uint2*>(slot + q * 8) = chunk_to_fp8(v[u], inv);
        }
    }
    __syncwarp();
    return scale;
}

// scale of a BF16 row in global memory (register path with rows that stay E4M3 at the receiver)
__device__ __forceinline__ float row_scale_from_global(const std::uint8_t* src, int hidden, bool vec_ok) {
    const unsigned lane = ptx::lane_id();
    float amax = 0.0f;
    if (vec_ok) {
        for (int q = lane; q < hidden / 8; q += 32) amax = fmaxf(amax, chunk_amax(ptx::ld_nc_v4(src + static_cast<std::size_t>(q) * 16)));
    } else {
        const auto* s = reinterpret_cast<const __nv_bfloat16*>(src);
        for (int i = lane; i < hidden; i += 32) amax = fmaxf(amax, fabsf(__bfloat162float(s[i])));
    }
    return fp8_scale_from_amax(warp_max(amax));
}

// Where one received row goes: computes its output rows, writes the per-row outputs (expert id, weight, source,
// scale) and the entry of the combine map, and leaves the pointer of output row i in lane i < n_rows.
// `e`, `ord`, `wgt` are per lane k.  Returns true (warp-uniform) when a row would fall outside its capacity.
__device__ __forceinline__ bool place_row(const Ctx& k, int s, int j, int token, float scale, int e, int ord, float wgt,
                                          std::uint8_t*& out_ptr, int& n_rows) {
    const DispatchArgs& a = *k.a;
    const unsigned lane = ptx::lane_id();
    const unsigned full = 0xffffffffu;
    const unsigned lt_mask = (1u << lane) - 1u;
    const bool local = e >= 0 && e / k.El == k.me;
    const int el = local ? e - k.me * k.El : -1;
    const unsigned lmask = __ballot_sync(full, local);
    const int n_local = __popc(lmask);
    const int pos = __popc(lmask & lt_mask);
    int* map = a.comb_map + ((static_cast<std::size_t>(s) * k.C + k.c) * k.Qf + j) * k.map_stride;
    out_ptr = nullptr;
    bool overflow = false;
    if (a.do_expand) {
        n_rows = n_local;
        int row = -1;
        if (local) {
            row = k.eoff[el] + k.spre[s * k.El + el] + ord;
            overflow = row < 0 || row >= k.expanded_cap;
        }
        // compact: the i-th local slot's row goes to lane i
        for (unsigned lm = lmask, i = 0; lm; lm &= lm - 1, ++i) {
            const int r = __shfl_sync(full, row, __ffs(lm) - 1);
            if (lane == i) out_ptr = k.recv_bytes + static_cast<std::size_t>(r) * k.out_row_bytes;
        }
        if (local && !overflow) {
            if (k.recv_fp8) a.recv_scale[row] = scale;
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
        const int row = k.sh->source_offsets[s] + k.sh->chan_base[s] + j;
        overflow = row < 0 || row >= k.unique_cap;
        if (lane == 0) out_ptr = k.recv_bytes + static_cast<std::size_t>(row) * k.out_row_bytes;
        if (!overflow) {
            if (k.recv_fp8 && lane == 0) a.recv_scale[row] = scale;
            if (lane < static_cast<unsigned>(k.K)) {
                a.recv_idx[static_cast<std::size_t>(row) * k.K + lane] = el;
                a.recv_w[static_cast<std::size_t>(row) * k.K + lane] = local ? wgt : 0.0f;
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
    return __any_sync(full, overflow) != 0;
}

}  // namespace detail

#endif  // __CUDACC__

}  // namespace bep
