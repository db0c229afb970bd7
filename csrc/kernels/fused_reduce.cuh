// Owner side of the combine paths: an ordinary (non-cooperative, fully occupied) launch.
//
// fused_reduce_kernel: producers on every rank have written weighted BF16 rows into this rank's landing area and
//   published their epoch; this kernel waits -- bounded -- for every rank's epoch, adds the rows of every token in
//   slot order (FP32, deterministic) and hands the area back.  Two producers use it:
//     * combine_push_kernel (combine_push.cuh): one slot per (token, expert rank), valid where the token's
//       destination mask has that rank's bit;
//     * the fused down projection (expert_gemm.cu, scatter variant): one slot per (token, k), valid where the
//       routing plan's expert ordinal is >= 0.
#pragma once

#include "protocol.cuh"

namespace bep {

constexpr int kFusedReduceThreads = 256;
// column groups per step of the owner-side reduction (see fused_reduce_kernel)
constexpr int fused_reduce_groups(int slots) { return slots <= 2 ? 4 : (slots <= 4 ? 2 : 1); }

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

// G = column groups (of 32 sixteen-byte chunks) a warp handles per step.  A step keeps eight row loads per lane in
// flight: eight slots of one group, or -- when a token has few slots, as with two or four ranks -- 8 / G slots of G
// groups each (measured at two ranks: 58 -> 43 us for the same rows).  The slots of an element are added in slot
// order whatever G is, so the result does not depend on it.
template <int G>
__global__ void __launch_bounds__(kFusedReduceThreads, G == 1 ? 4 : 3) fused_reduce_kernel(const FusedReduceArgs a) {
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
        const int steps_per_token = (groups + G - 1) / G;
        const long long units = static_cast<long long>(a.num_tokens) * steps_per_token;
        const long long total_warps = static_cast<long long>(gridDim.x) * warps;
        const long long me = static_cast<long long>(blockIdx.x) * warps + warp;
        const long long first = units * me / total_warps, last = units * (me + 1) / total_warps;
        const std::uint8_t* area = rc->seg[rc->rank] + a.stage_off;
        const std::size_t pitch = a.slot_stride;
        constexpr int kSlotsPerPass = 8 / G;
        int cached_token = -1;
        unsigned valid = 0;
        for (long long u = first; u < last; ++u) {
            const int t = static_cast<int>(u / steps_per_token);
            const int c0 = static_cast<int>(u % steps_per_token) * G * 32 + lane;  // this lane's chunk in the step's first group
            if (t != cached_token) {
                if (a.expert_ord != nullptr) {
                    const int ord = lane < K ? a.expert_ord[static_cast<std::size_t>(t) * K + lane] : -1;
                    valid = __ballot_sync(0xffffffffu, ord >= 0);
                } else {
                    valid = a.rank_mask[t];
                }
                cached_token = t;
            }
            const std::uint8_t* rows = area + static_cast<std::size_t>(t) * a.token_stride;
            float acc[G][8];
#pragma unroll
            for (int g = 0; g < G; ++g)
#pragma unroll
                for (int x = 0; x < 8; ++x) acc[g][x] = 0.f;
            for (int k0 = 0; k0 < K; k0 += kSlotsPerPass) {
                uint4 v[G][kSlotsPerPass];
#pragma unroll
                for (int g = 0; g < G; ++g) {
                    const int c = c0 + g * 32;
#pragma unroll
                    for (int j = 0; j < kSlotsPerPass; ++j) {
                        const int k = k0 + j;
                        v[g][j] = (c < chunks && k < K && (valid >> k & 1u)) ? ptx::ld_v4(rows + static_cast<std::size_t>(c) * 16 + k * pitch)
                                                                            : make_uint4(0u, 0u, 0u, 0u);
                    }
                }
#pragma unroll
                for (int g = 0; g < G; ++g)
#pragma unroll
                    for (int j = 0; j < kSlotsPerPass; ++j) fused_accumulate(acc[g], v[g][j]);
            }
#pragma unroll
            for (int g = 0; g < G; ++g) {
                const int c = c0 + g * 32;
                if (c < chunks) {
                    uint4 packed;
                    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
                    for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(acc[g][2 * j], acc[g][2 * j + 1]);
                    reinterpret_cast<uint4*>(a.out + static_cast<std::size_t>(t) * lay.hidden)[c] = packed;
                }
            }
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

#endif  // __CUDACC__

}  // namespace bep
