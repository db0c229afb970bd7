// Weighted combine in one cooperative launch per rank (`combine_reduce="inline"`): the inverse of a finished
// dispatch with the owner-side sum running in the same kernel, so a token's rows are added as they arrive.
// The default combine is the two ordinary launches of combine_push.cuh and fused_reduce.cuh; this kernel is the variant that starts
// the owner-side sum before the last row has been pushed, at the price of a cooperative launch.
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

// dst[q] = bf16( w * src[q] ): the single-row case of reduce_rows (the common one when a token reaches a rank
// through one expert only), eight 16-byte chunks per lane in flight instead of four.
__device__ __noinline__ void scale_row(const std::uint8_t* src, float w, std::uint8_t* dst, int chunks) {
    const unsigned lane = ptx::lane_id();
    for (int q0 = 0; q0 < chunks; q0 += 256) {
        uint4 v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int q = q0 + u * 32 + lane;
            if (q < chunks) v[u] = ptx::ld_v4(src + static_cast<std::size_t>(q) * 16);
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int q = q0 + u * 32 + lane;
            if (q < chunks) {
                float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                accumulate_chunk(acc, v[u], w);
                *reinterpret_cast<uint4*>(dst + static_cast<std::size_t>(q) * 16) = pack_chunk(acc);
            }
        }
    }
}

// dst[q] = bf16( sum_i w_i * rows_i[q] ) over `n` rows, FP32 accumulation in row order.  Row i lives at
// base + index(lane i) * stride, its weight in lane i.  `dst` is a generic pointer (shared or global).
// Rows are taken two at a time, four 16-byte chunks per lane each: 8 loads in flight per lane.
__device__ __forceinline__ void reduce_rows(const std::uint8_t* base, std::size_t stride, int index_of_lane,
                                            float weight_of_lane, int n, std::uint8_t* dst, int chunks) {
    const unsigned lane = ptx::lane_id();
    if (n == 1) {
        scale_row(base + static_cast<std::size_t>(__shfl_sync(0xffffffffu, index_of_lane, 0)) * stride,
                  __shfl_sync(0xffffffffu, weight_of_lane, 0), dst, chunks);
        return;
    }
    for (int q0 = 0; q0 < chunks; q0 += 128) {
        float acc[4][8];
#pragma unroll
        for (int u = 0; u < 4; ++u)
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[u][e] = 0.0f;
        for (int i0 = 0; i0 < n; i0 += 2) {
            const bool two = i0 + 1 < n;
            const std::uint8_t* src0 = base + static_cast<std::size_t>(__shfl_sync(0xffffffffu, index_of_lane, i0)) * stride;
            const std::uint8_t* src1 = base + static_cast<std::size_t>(__shfl_sync(0xffffffffu, index_of_lane, two ? i0 + 1 : i0)) * stride;
            const float w0 = __shfl_sync(0xffffffffu, weight_of_lane, i0);
            const float w1 = __shfl_sync(0xffffffffu, weight_of_lane, two ? i0 + 1 : i0);
            uint4 v0[4], v1[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int q = q0 + u * 32 + lane;
                if (q < chunks) {
                    v0[u] = ptx::ld_v4(src0 + static_cast<std::size_t>(q) * 16);
                    if (two) v1[u] = ptx::ld_v4(src1 + static_cast<std::size_t>(q) * 16);
                }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int q = q0 + u * 32 + lane;
                if (q < chunks) {
                    accumulate_chunk(acc[u], v0[u], w0);
                    if (two) accumulate_chunk(acc[u], v1[u], w1);
                }
            }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int q = q0 + u * 32 + lane;
            if (q < chunks) *reinterpret_cast<uint4*>(dst + static_cast<std::size_t>(q) * 16) = pack_chunk(acc[u]);
        }
    }
}

}  // namespace detail

// Each warp owns one row buffer in shared memory (the partial row it is about to push).
constexpr int kCombineWarps = 12;  // every warp first reduces+pushes expert-side rows, then adds rows for its own tokens

__global__ void __launch_bounds__(kCombineWarps * 32, 1) combine_kernel(const __grid_constant__ CombineLaunch launch) {
    using namespace detail;
    const CombineArgs& a = launch.r[blockIdx.y];
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
    // one rank: the reduced row of a token is already the result -- it goes straight to `out`, nothing is
    // staged and there is no owner-side pass
    const bool direct = P == 1 && vec_ok;
    __shared__ int cta_flag;
    __shared__ unsigned long long stat[4];
    extern __shared__ __align__(128) unsigned char row_buffers[];  // [warps][crow_stride] (vector-capable hidden only)
    unsigned char* my_buffer = row_buffers + static_cast<std::size_t>(warp) * lay.crow_stride;

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
    std::int64_t* prof = a.profile + static_cast<std::size_t>(c) * 8;
    if (threadIdx.x == 0) prof[0] = static_cast<std::int64_t>(ptx::globaltimer_ns());
    if (cta_failed(health, &cta_flag)) return;
    if (threadIdx.x == 0) {
        prof[1] = static_cast<std::int64_t>(ptx::globaltimer_ns());
        prof[2] = 0;
    }

    unsigned long long st_rows = 0, st_remote = 0, st_tokens = 0;
    {
        // Every warp walks one work list: first its share of the expert-side rows (reduce the local
        // expert outputs of one received token, push the partial row to the token's source; never waits),
        // then its share of this rank's own tokens (wait for the partial rows, add them in rank order).
        // Both kinds of work end in the same reduction code, instantiated once.
        const int w = warp;
        const std::size_t rank_stride = static_cast<std::size_t>(Tmax) * lay.crow_stride;
        // expert-side cursor.  Sources are visited in a rank-rotated order: at any moment every rank
        // pushes to a different peer instead of all ranks converging on source 0, then source 1, ...
        // expert-side cursor: rows are taken round-robin over the sources (row jj of every source in
        // turn, starting with rank me+1), so a rank sprays all its peers at once like dispatch does and
        // no destination is the target of every rank at the same time.
        int step = 0, jj = 0, item = 0, s = 0;
        const int my_count = lane < static_cast<unsigned>(P) ? a.recv_chan_counts[lane * C + c] : 0;
        int max_count = my_count;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) max_count = max(max_count, __shfl_xor_sync(full, max_count, o));
        int t = t0 + w;  // source-side cursor
        // A pushed row travels as one bulk copy from this warp's shared-memory buffer.  Its flag is
        // released one row late: after the next row's copy has been issued and the older bulk group has
        // completed (cp.async.bulk.wait_group 1), so the round trip to the peer overlaps the next row.
        std::uint64_t* pending_flag = nullptr;
        while (true) {
            const std::uint8_t* row_base = nullptr;  // row i of the reduction = row_base + row_index(lane i) * row_stride
            std::size_t row_stride = 0;
            int row_index = 0;
            float wgt = 1.0f;
            int n = 0;
            std::uint8_t* dst = nullptr;
            std::uint64_t* flag = nullptr;
            bool coherent_side = false;
            // ---- next expert-side item of this warp
            bool have = false;
            int j = 0;
            while (jj < max_count && !have) {
                if (step >= P) {
                    step = 0;
                    ++jj;
                    continue;
                }
                s = (me + 1 + step) % P;
                const int n_s = __shfl_sync(full, my_count, s);
                ++step;
                if (jj < n_s) {
                    if (item % num_warps == w) {
                        have = true;
                        j = jj;
                    }
                    ++item;
                }
            }
            if (have) {
                const int* map = a.comb_map + ((static_cast<std::size_t>(s) * C + c) * Qf + j) * map_stride;
                const int token = map[0];
                n = map[1];
                row_base = reinterpret_cast<const std::uint8_t*>(a.y);
                row_stride = static_cast<std::size_t>(H) * 2;
                if (static_cast<int>(lane) < n) {
                    row_index = map[2 + 2 * lane];
                    wgt = a.weighted ? __int_as_float(map[3 + 2 * lane]) : 1.0f;
                }
                dst = rc->seg[s] + lay.cstage_off + static_cast<std::size_t>(me) * rank_stride +
                      static_cast<std::size_t>(token) * lay.crow_stride;
                flag = reinterpret_cast<std::uint64_t*>(rc->seg[s] + lay.cready_off) + static_cast<std::size_t>(me) * Tmax + token;
                if (direct) dst = reinterpret_cast<std::uint8_t*>(a.out + static_cast<std::size_t>(token) * H);
                if (lane == 0) {
                    ++st_rows;
                    if (s != me) ++st_remote;
                }
            } else {
                // ---- next own token of this warp.  Nothing of the expert side may stay unpublished while
                // this warp waits for its peers (they wait for exactly those rows).
                if (pending_flag != nullptr) {
                    if (lane == 0) {
                        ptx::bulk_wait_all();
                        if (!direct) ptx::st_release_sys(pending_flag, epoch);
                    }
                    pending_flag = nullptr;
                }
                if (warp == 0 && lane == 0 && prof[2] == 0) prof[2] = static_cast<std::int64_t>(ptx::globaltimer_ns());
                if (direct) {
                    // tokens that were routed nowhere get no row from the expert side: their result is zero
                    for (int tz = t0 + w; tz < t1; tz += num_warps) {
                        if (a.plan_mask[tz] != 0) continue;
                        uint4* row = reinterpret_cast<uint4*>(a.out + static_cast<std::size_t>(tz) * H);
                        for (int q = lane; q < H / 8; q += 32) row[q] = make_uint4(0u, 0u, 0u, 0u);
                    }
                    break;
                }
                if (t >= t1) break;
                const unsigned mask = a.plan_mask[t];
                if (lane < static_cast<unsigned>(P) && (mask >> lane & 1u)) {
                    const std::uint64_t* ready = reinterpret_cast<const std::uint64_t*>(my_seg + lay.cready_off) +
                                                 static_cast<std::size_t>(lane) * Tmax + t;
                    while (ptx::ld_acquire_sys(ready) != epoch) {
                        if (health.give_up(kErrRowWait, lane, t)) break;
                    }
                }
                __syncwarp();
                coherent_side = true;
                row_base = my_seg + lay.cstage_off + static_cast<std::size_t>(t) * lay.crow_stride;
                row_stride = rank_stride;
                unsigned m = mask;
                for (unsigned i = 0; m; m &= m - 1, ++i)
                    if (lane == i) row_index = __ffs(m) - 1;
                n = __popc(mask);
                dst = reinterpret_cast<std::uint8_t*>(a.out + static_cast<std::size_t>(t) * H);
                t += num_warps;
                if (lane == 0) ++st_tokens;
            }
            if (warp_failed(health)) break;
            if (vec_ok && flag != nullptr) {
                if (lane == 0) ptx::bulk_wait_read_all();  // the previous copy has left the buffer
                __syncwarp();
                reduce_rows(row_base, row_stride, row_index, wgt, n, my_buffer, H / 8);
                ptx::fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                    ptx::bulk_s2g(dst, my_buffer, static_cast<unsigned>(H) * 2);
                    ptx::bulk_commit();
                    if (pending_flag != nullptr && !direct) {
                        asm volatile("cp.async.bulk.wait_group 1;" ::: "memory");
                        ptx::st_release_sys(pending_flag, epoch);
                    }
                }
                pending_flag = flag;
                continue;
            } else if (vec_ok) {
                reduce_rows(row_base, row_stride, row_index, wgt, n, dst, H / 8);
            } else {
                for (int k = lane; k < H; k += 32) {
                    float acc = 0.0f;
                    for (int i = 0; i < n; ++i) {
                        const auto* src = reinterpret_cast<const volatile std::uint16_t*>(
                            row_base + static_cast<std::size_t>(__shfl_sync(full, row_index, i)) * row_stride);
                        const float wi = __shfl_sync(full, wgt, i);
                        const std::uint16_t bits = src[k];
                        acc = fmaf(wi, __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(&bits)), acc);
                    }
                    reinterpret_cast<__nv_bfloat16*>(dst)[k] = __float2bfloat16_rn(acc);
                }
            }
            (void)coherent_side;
            if (flag != nullptr) {
                __syncwarp();
                if (lane == 0) ptx::st_release_sys(flag, epoch);
            }
        }
        if (lane == 0) {
            ptx::bulk_wait_all();
            if (pending_flag != nullptr && !direct) ptx::st_release_sys(pending_flag, epoch);
        }
    }

    __syncwarp();
    if (warp == 0 && lane == 0) prof[3] = static_cast<std::int64_t>(ptx::globaltimer_ns());
    if (lane == 0) {
        atomicAdd(&stat[0], st_rows);
        atomicAdd(&stat[1], st_remote);
        atomicAdd(&stat[2], st_tokens);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        prof[4] = static_cast<std::int64_t>(ptx::globaltimer_ns());
        const int stat_base = C + rc->send_ctas;  // second half of the per-CTA statistics: combine
        std::int64_t* cs = rc->chan_stats + static_cast<std::size_t>(stat_base + c) * 10;
        for (int i = 0; i < 3; ++i) cs[i] = static_cast<std::int64_t>(stat[i]);
        __threadfence();
        const unsigned long long old = atomicAdd(&rc->done_ctas[1], 1ull);
        if ((old + 1) % static_cast<unsigned long long>(C) == 0) {
            __threadfence();
            std::int64_t sum[3] = {0, 0, 0};
            for (int c2 = 0; c2 < C; ++c2)
                for (int i = 0; i < 3; ++i) sum[i] += __ldcg(rc->chan_stats + static_cast<std::size_t>(stat_base + c2) * 10 + i);
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
