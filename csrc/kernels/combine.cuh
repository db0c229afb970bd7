// Fused weighted combine: the inverse of a finished dispatch, one cooperative launch per rank.
// The reference stops at dispatch (pcie_ep/buffers/ep.py:461-462 raises); its design note
// (docs/pcie-ep/design.md:420-422) sketches this inverse: reduce on the expert rank what belongs to one
// source token, send one row per (token, expert rank) back, add the partial rows at the source.
//
// Expert side (send warps): for every row this rank received in the dispatch (the dispatch left an
// inverse map: source token, output rows, weights) reduce the expert outputs of that token with the
// dispatch-time weights in FP32, round to BF16 and store the row straight into the source rank's
// combine area over NVLink, then release that (expert rank, token) flag there.
// Source side (reduce warps): for every own token wait (locally) for the flags of the ranks in the
// token's destination mask and add their rows in rank order in FP32.
// The order of floating-point operations is fixed, so the result is deterministic.
#pragma once

#include "dispatch.cuh"

namespace bep {

#ifdef __CUDACC__

namespace detail {

__device__ __forceinline__ void accumulate_chunk(float (&acc)[8], const uint4& v, float w) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(h[i]);
        acc[2 * i] = fmaf(w, f.x, acc[2 * i]);
        acc[2 * i + 1] = fmaf(w, f.y, acc[2 * i + 1]);
    }
}
__device__ __forceinline__ uint4 pack_chunk(const float (&acc)[8]) {
    uint4 out;
    __nv_bfloat162* o = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
    for (int i = 0; i < 4; ++i) o[i] = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
    return out;
}

// dst[q] = bf16( sum_i w_i * rows_i[q] ) over `n` rows, FP32 accumulation in row order.  Lane i < n
// holds row i's pointer and weight.  One pass keeps ROWS x CH 16-byte loads in flight per lane (64
// registers of payload) before the first is consumed; the caller picks the shape from n.
// n <= ROWS: the sum of one chunk is formed in one go, nothing is carried between passes.
template <int ROWS, int CH, bool COHERENT>
__device__ __forceinline__ void reduce_rows_once(const std::uint8_t* row_of_lane, float weight_of_lane, int n,
                                                 std::uint8_t* dst, int chunks) {
    const unsigned lane = ptx::lane_id();
    const std::uint8_t* src[ROWS];
    float w[ROWS];
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
        src[r] = shfl_ptr(const_cast<std::uint8_t*>(row_of_lane), r);
        w[r] = __shfl_sync(0xffffffffu, weight_of_lane, r);
    }
    for (int q0 = 0; q0 < chunks; q0 += 32 * CH) {
        uint4 v[ROWS][CH];
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            if (r < n) {
#pragma unroll
                for (int u = 0; u < CH; ++u) {
                    const int q = q0 + u * 32 + lane;
                    if (q < chunks)
                        v[r][u] = COHERENT ? ptx::ld_v4(src[r] + static_cast<std::size_t>(q) * 16)
                                           : ptx::ld_nc_v4(src[r] + static_cast<std::size_t>(q) * 16);
                }
            }
        }
#pragma unroll
        for (int u = 0; u < CH; ++u) {
            const int q = q0 + u * 32 + lane;
            if (q < chunks) {
                float acc[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                for (int r = 0; r < ROWS; ++r)
                    if (r < n) accumulate_chunk(acc, v[r][u], w[r]);
                ptx::st_v4(dst + static_cast<std::size_t>(q) * 16, pack_chunk(acc));
            }
        }
    }
}

// any n: rows in groups of 8, partial sums carried in registers
template <bool COHERENT>
__device__ __forceinline__ void reduce_rows_many(const std::uint8_t* row_of_lane, float weight_of_lane, int n,
                                                 std::uint8_t* dst, int chunks) {
    const unsigned lane = ptx::lane_id();
    for (int q0 = 0; q0 < chunks; q0 += 64) {
        float acc[2][8];
#pragma unroll
        for (int u = 0; u < 2; ++u)
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[u][e] = 0.0f;
        for (int i0 = 0; i0 < n; i0 += 4) {
            uint4 v[4][2];
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                if (i0 + r < n) {
                    const std::uint8_t* src = shfl_ptr(const_cast<std::uint8_t*>(row_of_lane), i0 + r);
#pragma unroll
                    for (int u = 0; u < 2; ++u) {
                        const int q = q0 + u * 32 + lane;
                        if (q < chunks)
                            v[r][u] = COHERENT ? ptx::ld_v4(src + static_cast<std::size_t>(q) * 16)
                                               : ptx::ld_nc_v4(src + static_cast<std::size_t>(q) * 16);
                    }
                }
            }
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                if (i0 + r < n) {
                    const float w = __shfl_sync(0xffffffffu, weight_of_lane, i0 + r);
#pragma unroll
                    for (int u = 0; u < 2; ++u) {
                        const int q = q0 + u * 32 + lane;
                        if (q < chunks) accumulate_chunk(acc[u], v[r][u], w);
                    }
                }
            }
        }
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int q = q0 + u * 32 + lane;
            if (q < chunks) ptx::st_v4(dst + static_cast<std::size_t>(q) * 16, pack_chunk(acc[u]));
        }
    }
}

template <bool COHERENT>
__device__ __forceinline__ void reduce_rows_any(const std::uint8_t* row_of_lane, float weight_of_lane, int n,
                                                std::uint8_t* dst, int chunks) {
    if (n <= 2) reduce_rows_once<2, 4, COHERENT>(row_of_lane, weight_of_lane, n, dst, chunks);
    else if (n <= 8) reduce_rows_once<8, 1, COHERENT>(row_of_lane, weight_of_lane, n, dst, chunks);
    else reduce_rows_many<COHERENT>(row_of_lane, weight_of_lane, n, dst, chunks);
}

}  // namespace detail

constexpr int kCombineWarps = 10;  // every warp first reduces+pushes expert-side rows, then adds rows for its own tokens

__global__ void __launch_bounds__(kCombineWarps * 32, 1) combine_kernel(const __grid_constant__ CombineLaunch launch) {
    using namespace detail;
    const CombineArgs a = launch.r[blockIdx.y];
    const RankConst* __restrict__ rc = a.rc;
    const SegmentLayout& lay = rc->lay;
    const int P = lay.num_ranks, C = lay.num_channels, K = lay.num_topk, H = lay.hidden, Qf = lay.slots_full;
    const int Tmax = lay.num_max_tokens;
    const int me = rc->rank, c = blockIdx.x;
    const int T = a.num_tokens;
    const int Tc = (T + C - 1) / C;
    const int t0 = min(T, c * Tc), t1 = min(T, t0 + Tc);
    const int warp = threadIdx.x >> 5;
    const unsigned lane = ptx::lane_id();
    const unsigned full = 0xffffffffu;
    const int num_warps = blockDim.x >> 5;
    const bool vec_ok = rc->vec_ok != 0;
    const int map_stride = 2 + 2 * K;
    __shared__ int cta_flag;
    __shared__ unsigned long long stat[4];

    Health health(rc, a.error);
    const std::uint64_t epoch = rc->epochs[1] + 1;
    std::uint8_t* my_seg = rc->seg[me];

    if (ptx::ld_volatile(&rc->sticky[0]) != 0) {
        if (threadIdx.x == 0 && c == 0) atomicCAS(&a.error[0], 0, kErrAlreadyAborted);
        return;
    }
    if (threadIdx.x < 4) stat[threadIdx.x] = 0;
    // reuse guard: a source must have finished adding the previous combine's rows before new ones land
    if (warp == 0 && lane < static_cast<unsigned>(P)) {
        const std::uint64_t* done = flag_ptr(my_seg, lay.cdone_off, lane);
        while (ptx::ld_acquire_sys(done) + 1 < epoch) {
            if (health.give_up(kErrReuseGuardWait, lane, 1)) break;
        }
    }
    if (cta_failed(health, &cta_flag)) return;

    unsigned long long st_rows = 0, st_remote = 0, st_tokens = 0;
    {
        // ===== expert side: reduce + push (never waits) =====
        const int w = warp;
        int item = 0;
        // Destinations are visited in a rank-rotated order: at any moment every rank pushes to a
        // different peer, instead of all ranks converging on source 0 first, then source 1, ...
        for (int step = 0; step < P && !warp_failed(health); ++step) {
            const int s = (me + 1 + step) % P;
            const int n_s = a.recv_chan_counts[s * C + c];
            std::uint8_t* dst_base = rc->seg[s] + lay.cstage_off + static_cast<std::size_t>(me) * Tmax * lay.crow_stride;
            std::uint64_t* flag_base = reinterpret_cast<std::uint64_t*>(rc->seg[s] + lay.cready_off) + static_cast<std::size_t>(me) * Tmax;
            for (int j = 0; j < n_s; ++j, ++item) {
                if (item % num_warps != w) continue;
                const int* map = a.comb_map + ((static_cast<std::size_t>(s) * C + c) * Qf + j) * map_stride;
                const int token = map[0];
                const int n = map[1];
                const std::uint8_t* row_ptr = nullptr;
                float wgt = 0.0f;
                if (static_cast<int>(lane) < n) {
                    row_ptr = reinterpret_cast<const std::uint8_t*>(a.y + static_cast<std::size_t>(map[2 + 2 * lane]) * H);
                    wgt = a.weighted ? __int_as_float(map[3 + 2 * lane]) : 1.0f;
                }
                std::uint8_t* dst = dst_base + static_cast<std::size_t>(token) * lay.crow_stride;
                if (vec_ok) {
                    reduce_rows_any<false>(row_ptr, wgt, n, dst, H / 8);
                } else {
                    for (int k = lane; k < H; k += 32) {
                        float acc = 0.0f;
                        for (int i = 0; i < n; ++i) {
                            const auto* src = reinterpret_cast<const __nv_bfloat16*>(shfl_ptr(const_cast<std::uint8_t*>(row_ptr), i));
                            const float wi = __shfl_sync(full, wgt, i);
                            acc = fmaf(wi, __bfloat162float(src[k]), acc);
                        }
                        reinterpret_cast<__nv_bfloat16*>(dst)[k] = __float2bfloat16_rn(acc);
                    }
                }
                __syncwarp();
                if (lane == 0) {
                    ptx::st_release_sys(flag_base + token, epoch);
                    ++st_rows;
                    if (s != me) ++st_remote;
                }
            }
        }
    }
    {
        // ===== source side: add the partial rows of every destination rank, in rank order =====
        const int w = warp;
        for (int t = t0 + w; t < t1; t += num_warps) {
            if (warp_failed(health)) break;
            const unsigned mask = a.plan_mask[t];
            if (lane < static_cast<unsigned>(P) && (mask >> lane & 1u)) {
                const std::uint64_t* flag = reinterpret_cast<const std::uint64_t*>(my_seg + lay.cready_off) +
                                            static_cast<std::size_t>(lane) * Tmax + t;
                while (ptx::ld_acquire_sys(flag) != epoch) {
                    if (health.give_up(kErrRowWait, lane, t)) break;
                }
            }
            __syncwarp();
            if (warp_failed(health)) break;
            std::uint8_t* out = reinterpret_cast<std::uint8_t*>(a.out + static_cast<std::size_t>(t) * H);
            const std::uint8_t* base = my_seg + lay.cstage_off + static_cast<std::size_t>(t) * lay.crow_stride;
            const std::size_t rank_stride = static_cast<std::size_t>(Tmax) * lay.crow_stride;
            if (vec_ok) {
                // lane i holds the row of the i-th rank (ascending) in the token's mask
                const std::uint8_t* src_of_lane = nullptr;
                {
                    unsigned m = mask;
                    for (unsigned i = 0; m; m &= m - 1, ++i)
                        if (lane == i) src_of_lane = base + static_cast<std::size_t>(__ffs(m) - 1) * rank_stride;
                }
                reduce_rows_any<true>(src_of_lane, 1.0f, __popc(mask), out, H / 8);
            } else {
                for (int k = lane; k < H; k += 32) {
                    float acc = 0.0f;
                    for (unsigned m = mask; m; m &= m - 1) {
                        const auto* src = reinterpret_cast<const volatile std::uint16_t*>(base + static_cast<std::size_t>(__ffs(m) - 1) * rank_stride);
                        const std::uint16_t bits = src[k];
                        acc += __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(&bits));
                    }
                    reinterpret_cast<__nv_bfloat16*>(out)[k] = __float2bfloat16_rn(acc);
                }
            }
            if (lane == 0) ++st_tokens;
        }
    }

    __syncwarp();
    if (lane == 0) {
        atomicAdd(&stat[0], st_rows);
        atomicAdd(&stat[1], st_remote);
        atomicAdd(&stat[2], st_tokens);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        std::int64_t* cs = rc->chan_stats + static_cast<std::size_t>(C + c) * 10;  // second half: combine
        for (int i = 0; i < 3; ++i) cs[i] = static_cast<std::int64_t>(stat[i]);
        __threadfence();
        const unsigned long long old = atomicAdd(&rc->done_ctas[1], 1ull);
        if ((old + 1) % static_cast<unsigned long long>(C) == 0) {
            __threadfence();
            std::int64_t sum[3] = {0, 0, 0};
            for (int c2 = 0; c2 < C; ++c2)
                for (int i = 0; i < 3; ++i) sum[i] += __ldcg(rc->chan_stats + static_cast<std::size_t>(C + c2) * 10 + i);
            for (int i = 0; i < 8; ++i) a.stats[i] = i < 3 ? sum[i] : 0;
            if (!health.failed()) {
                for (int p = 0; p < P; ++p) ptx::st_release_sys(flag_ptr(rc->seg[p], lay.cdone_off, me), epoch);
            }
            rc->epochs[1] = epoch;
        }
    }
}

#endif  // __CUDACC__

}  // namespace bep
