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
    bool fence_flags, corrupt_sequence;
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
// which store the flags (`st.relaxed.sys`).  (With one fence per row -- host segments, or the conservative setting
// for peer segments -- every lane executes the fence after the `__syncwarp()` instead, so that the fence and the flag
// store it orders are in one thread.)  On this hardware such a fence waits for every store the SM still has
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
                    if (!fence_flags) ptx::fence_sys();
                }
                __syncwarp();
                if (fence_flags) ptx::fence_sys();  // (see the note on the two chains below)
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
        // With one fence per row (`fence_flags`: host segments, or the conservative setting for peer segments) every
        // lane fences after the barrier, so that the fence and the flag store it orders are in the same thread: the
        // release pattern as the memory model spells it.
        if (since_flags >= flag_batch && n >= kFlagLag) {
            BEP_ROLE_T(t_store);
            if (issuer) {
                bulk_wait_group<kFlagLag>();
                if (!fence_flags) ptx::fence_sys();
            }
            __syncwarp();
            if (fence_flags) ptx::fence_sys();
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
            if (!fence_flags) ptx::fence_sys();
        }
        __syncwarp();
        if (fence_flags) ptx::fence_sys();
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
