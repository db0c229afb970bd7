// Grouped expert GEMM for the expanded dispatch layout, on the 5th-generation tensor cores:
// tcgen05.mma issued by one elected thread, operands staged in shared memory by TMA
// (cp.async.bulk.tensor, no multicast), FP32 accumulators in tensor memory (TMEM), read back with
// tcgen05.ld for a fused epilogue.  The reference has no expert GEMM at all (docs/pcie-ep/design.md:304
// puts it out of scope); this is the "grouped SwiGLU expert FFN" that sits between dispatch and combine.
//
//   rows of expert e = A[expert_offsets[e] .. expert_offsets[e] + expert_counts[e])   (device-side ints)
//   plain  : out[row, n]        = sum_k A[row, k] * W[e, n, k]
//   SwiGLU : out[row, n]        = silu(sum_k A[row,k] * W[e, n, k]) * (sum_k A[row,k] * W[e, N + n, k])
//
// One tcgen05.mma covers 128 rows x 256 columns (two 128-row weight boxes back to back in shared memory:
// gate + up rows for SwiGLU, 256 adjacent output columns for the plain GEMM when n allows), so A is read
// from shared memory once per 256 accumulator columns.
//
// Work decomposition: persistent CTAs walk a tile list (expert, n-tile, m-tile) computed on the
// device from the counts -- the host never reads a count.  Per CTA: warp 0 = TMA producer,
// warp 1 = MMA issuer (and TMEM owner), warps 2..5 = epilogue.  Shared-memory stages are handed over
// with mbarriers (TMA complete_tx -> MMA; tcgen05.commit -> producer), accumulators are double
// buffered in TMEM (tcgen05.commit -> epilogue; epilogue arrive -> MMA).
//
// Every mbarrier wait is bounded: on expiry the thread latches an abort flag, all roles drain, TMEM
// is released and the kernel returns with status[0] != 0.
#pragma once

#include <cstdint>

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

namespace bep {
namespace gemm {

constexpr int kBlockM = 128;
constexpr int kBlockN = 128;
constexpr int kBlockKBytes = 128;  // one 128B-swizzle atom row: 64 bf16 or 128 fp8 elements of K
constexpr int kUmmaKBytes = 32;    // K extent of one tcgen05.mma: 16 bf16 or 32 fp8
constexpr int kThreads = 192;  // 6 warps
constexpr std::uint32_t kWaitLimit = 20u * 1000u * 1000u;  // try_wait probes before giving up (seconds at most)

// Fused down-projection + combine send: instead of writing `out`, the epilogue multiplies every valid row by
// its routing weight and stores it into the slot (token, k) of the token owner's landing area -- local memory or
// a peer's, through the segment table -- so the NVLink transfer of a tile overlaps the MMAs of the next ones.
// When the last CTA of the launch has drained its stores it publishes `epoch` to every rank.
constexpr int kScatterMaxRanks = 16;
constexpr int kScatterRowPitch = kBlockN * 2 + 16;  // one 128-column BF16 row segment + 16 B: conflict-free column writes
constexpr int kScatterStagingBytes = 4 * 32 * kScatterRowPitch;
struct ScatterTarget {
    unsigned char* seg[kScatterMaxRanks];  // segment of every rank as addressed from this one
    const long long* source_meta;          // [rows][3]: owner rank, token, slot k (-1: padding row)
    const float* row_weights;              // [rows] routing weight of the row; nullptr: 1
    unsigned long long stage_off, sig_off, done_off;  // landing area, "rows are here" flags, "area consumed" flags
    unsigned long long epoch;              // number of this fused call (1, 2, ...), the same on every rank
    unsigned long long* cta_done;          // local monotonic count of finished CTAs over all launches
    unsigned long long timeout_ns;
    int row_stride;                        // bytes between landing slots
    int num_topk, num_ranks, rank, flag_stride;
};

struct GroupedGemmParams {
    const int* expert_offsets;  // [E+1] first row of every expert in A / out
    const int* expert_counts;   // [E]   valid rows
    __nv_bfloat16* out;         // [rows, N]
    const float* a_scales;      // FP8 only: one scale per row of A
    const float* w_scales;      // FP8 only: one scale per weight row [E, (2)N]
    int* status;                // [4]: 0 = ok, 1 = a wait expired, 2 = shared memory misaligned, 3 = a peer never freed its area
    int num_experts;
    int n;                      // output columns
    int k;                      // reduction length in elements
    int rows_capacity;          // rows of A / out
    ScatterTarget scatter;      // only read by the scatter variant
};

// stages of (A tile + B boxes) that fit; a stage carries one or two 128-row weight boxes
template <int kBoxesB>
struct SmemPlan {
    static constexpr int kTileA = kBlockM * kBlockKBytes;
    static constexpr int kTileB = kBlockN * kBlockKBytes;
    static constexpr int kStageBytes = kTileA + kBoxesB * kTileB;
    static constexpr int kStages = kBoxesB == 2 ? 4 : 6;
    static constexpr int kBytes = kStages * kStageBytes + 1024 /* alignment slack */ + 256 /* barriers */;
};

}  // namespace gemm
}  // namespace bep
