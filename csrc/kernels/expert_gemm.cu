// tcgen05 grouped expert GEMM: device code and launcher.  See expert_gemm.cuh for the design.
#include "expert_gemm.cuh"

#include <mutex>

#include "expert_gemm.hpp"
#include "ptx.cuh"

namespace bep {
namespace gemm {

namespace {

// ---- PTX wrappers ---------------------------------------------------------------------------
__device__ __forceinline__ std::uint32_t smem_addr(const void* p) {
    return static_cast<std::uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(std::uint64_t* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(std::uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(std::uint64_t* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(std::uint64_t* bar, unsigned parity) {
    std::uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_addr(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// bounded wait; returns false (and latches *abort) when the limit is hit or somebody else aborted
__device__ __forceinline__ bool mbar_wait(std::uint64_t* bar, unsigned parity, volatile int* abort) {
    for (std::uint32_t i = 0; i < kWaitLimit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 1023u) == 1023u && *abort) return false;
    }
    *abort = 1;
    return false;
}

// 2-D tiled TMA load, no multicast: box lands in shared memory with the tensor map's swizzle
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int x, int y, std::uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_addr(smem_dst)), "l"(reinterpret_cast<std::uint64_t>(map)), "r"(x), "r"(y), "r"(smem_addr(bar))
        : "memory");
}

__device__ __forceinline__ void tmem_alloc(std::uint32_t* smem_result, unsigned columns) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(smem_result)), "r"(columns)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(std::uint32_t taddr, unsigned columns) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(columns) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// D[tmem] (+)= A[smem desc] * B[smem desc]; one thread issues for the CTA
__device__ __forceinline__ void umma_f16(std::uint32_t tmem_d, std::uint64_t desc_a, std::uint64_t desc_b,
                                         std::uint32_t idesc, std::uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_f8(std::uint32_t tmem_d, std::uint64_t desc_a, std::uint64_t desc_b,
                                        std::uint32_t idesc, std::uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
// all MMAs issued so far by this thread arrive on `bar` when they have completed
__device__ __forceinline__ void umma_commit(std::uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_addr(bar))
                 : "memory");
}
// 32 lanes x 32 columns of FP32 out of TMEM: thread i gets columns [c, c+32) of lane (base lane + i)
__device__ __forceinline__ void tmem_ld_32x32(std::uint32_t taddr, std::uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes (64 bf16) wide, stored
// with the 128-byte swizzle TMA applied: 8-row groups are 1024 bytes apart (stride byte offset), the
// leading byte offset is unused for swizzled K-major operands, descriptor version 1 (sm_100),
// layout type 2 = SWIZZLE_128B.
__device__ __forceinline__ std::uint64_t make_smem_desc(const void* tile) {
    const std::uint64_t addr = smem_addr(tile);
    std::uint64_t desc = 0;
    desc |= (addr & 0x3FFFFull) >> 4;                 // bits  0..13 start address / 16
    desc |= static_cast<std::uint64_t>(0) << 16;      // bits 16..29 leading byte offset / 16
    desc |= static_cast<std::uint64_t>(1024 >> 4) << 32;  // bits 32..45 stride byte offset / 16
    desc |= static_cast<std::uint64_t>(1) << 46;      // bits 46..47 descriptor version
    desc |= static_cast<std::uint64_t>(2) << 61;      // bits 61..63 swizzle mode: 128B
    return desc;
}

// Instruction descriptor, kind::f16: D = F32, A = B = BF16, both K-major, N and M encoded /8 and /16.
__host__ __device__ constexpr std::uint32_t make_idesc_bf16(int m, int n) {
    return (1u << 4)                                   // D format: F32
           | (1u << 7)                                 // A format: BF16
           | (1u << 10)                                // B format: BF16
           | (static_cast<std::uint32_t>(n >> 3) << 17)
           | (static_cast<std::uint32_t>(m >> 4) << 24);
}

// kind::f8f6f4 with E4M3 operands (format code 0 for both), FP32 accumulation
__host__ __device__ constexpr std::uint32_t make_idesc_e4m3(int m, int n) {
    return (1u << 4) | (static_cast<std::uint32_t>(n >> 3) << 17) | (static_cast<std::uint32_t>(m >> 4) << 24);
}

struct TileCursor {
    // walks tiles in (expert, n-tile, m-tile) order: consecutive tiles share the weight tile
    int expert = 0;
    int first_tile = 0;  // index of the expert's first tile
    int m_tiles = 0;

    __device__ __forceinline__ bool locate(int tile, const GroupedGemmParams& p, int n_tiles, int& m_tile, int& n_tile) {
        while (expert < p.num_experts) {
            m_tiles = (p.expert_counts[expert] + kBlockM - 1) / kBlockM;
            const int tiles_here = m_tiles * n_tiles;
            if (tile < first_tile + tiles_here) {
                const int local = tile - first_tile;
                n_tile = local / m_tiles;
                m_tile = local % m_tiles;
                return true;
            }
            first_tile += tiles_here;
            ++expert;
        }
        return false;
    }
};

}  // namespace

// kBoxesB: 128-row weight boxes per stage.  Two boxes land back to back in shared memory and feed ONE
// tcgen05.mma of N = 256 (A is read from shared memory once per 256 output columns): for SwiGLU they are
// the gate and the up rows of the same 128 output columns, for the plain GEMM 256 adjacent output columns.
template <bool kSwiGLU, bool kFp8, int kBoxesB, bool kScatter>
__global__ void __launch_bounds__(kThreads, 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const GroupedGemmParams p) {
    static_assert(kBoxesB == 2 || !kSwiGLU, "SwiGLU stages carry the gate and the up box");
    static_assert(!kScatter || (kBoxesB == 2 && !kSwiGLU && !kFp8), "the scatter epilogue exists for the plain BF16 256-column tile");
    using Plan = SmemPlan<kBoxesB>;
    constexpr int kStages = Plan::kStages;
    constexpr int kAccCols = kBoxesB * kBlockN;   // TMEM columns of one accumulator set = N of one MMA
    constexpr int kTmemCols = 2 * kAccCols;       // double buffered: 256 or 512 (powers of two)
    constexpr int kOutN = kSwiGLU ? kBlockN : kAccCols;  // output columns of one tile

    extern __shared__ __align__(1024) unsigned char smem_unaligned[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<std::uintptr_t>(smem_unaligned) + 1023) & ~std::uintptr_t(1023));
    if (kScatter) {
        // the scatter variant asks for less alignment slack than the worst case: refuse (uniformly) instead of overrunning
        std::uint32_t dynamic_bytes;
        asm volatile("mov.u32 %0, %%dynamic_smem_size;" : "=r"(dynamic_bytes));
        const std::uint32_t needed = static_cast<std::uint32_t>(smem - smem_unaligned) + kStages * Plan::kStageBytes + 256 + kScatterStagingBytes;
        if (needed > dynamic_bytes) {
            if (threadIdx.x == 0) atomicExch(&p.status[0], 2);
            return;
        }
    }
    unsigned char* staging = smem + kStages * Plan::kStageBytes + 256;
    unsigned char* tiles = smem;
    std::uint64_t* full_bar = reinterpret_cast<std::uint64_t*>(smem + kStages * Plan::kStageBytes);
    std::uint64_t* empty_bar = full_bar + kStages;
    std::uint64_t* tmem_full = empty_bar + kStages;
    std::uint64_t* tmem_empty = tmem_full + 2;
    std::uint32_t* tmem_ptr = reinterpret_cast<std::uint32_t*>(tmem_empty + 2);
    volatile int* abort = reinterpret_cast<volatile int*>(tmem_ptr + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    constexpr int kElemBytes = kFp8 ? 1 : 2;
    constexpr int kBlockK = kBlockKBytes / kElemBytes;  // elements of K per stage
    const int n_tiles = p.n / kOutN;
    const int k_blocks = p.k / kBlockK;
    const int w_rows_per_expert = kSwiGLU ? 2 * p.n : p.n;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&tmem_full[b], 1);
            mbar_init(&tmem_empty[b], 4);
        }
        *abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        tmem_alloc(tmem_ptr, kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const std::uint32_t tmem_base = *tmem_ptr;

    if (warp == 0) {
        // ===== TMA producer =====
        if (lane == 0) {
            TileCursor cursor;
            int stage = 0;
            unsigned phase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok; tile += gridDim.x) {
                int m_tile, n_tile;
                if (!cursor.locate(tile, p, n_tiles, m_tile, n_tile)) break;
                const int row0 = p.expert_offsets[cursor.expert] + m_tile * kBlockM;
                const int wrow0 = cursor.expert * w_rows_per_expert + n_tile * kOutN;
                const int wrow1 = wrow0 + (kSwiGLU ? p.n : kBlockN);
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!mbar_wait(&empty_bar[stage], phase ^ 1u, abort)) {
                        ok = false;
                        break;
                    }
                    unsigned char* stage_base = tiles + stage * Plan::kStageBytes;
                    mbar_expect_tx(&full_bar[stage], Plan::kStageBytes);
                    tma_load_2d(stage_base, &map_a, kb * kBlockK, row0, &full_bar[stage]);
                    tma_load_2d(stage_base + Plan::kTileA, &map_b, kb * kBlockK, wrow0, &full_bar[stage]);
                    if (kBoxesB == 2)
                        tma_load_2d(stage_base + Plan::kTileA + Plan::kTileB, &map_b, kb * kBlockK, wrow1, &full_bar[stage]);
                    if (++stage == kStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ===== MMA issuer =====
        if (lane == 0) {
            constexpr std::uint32_t idesc = kFp8 ? make_idesc_e4m3(kBlockM, kAccCols) : make_idesc_bf16(kBlockM, kAccCols);
            TileCursor cursor;
            int stage = 0;
            unsigned phase = 0;
            bool ok = true;
            int it = 0;
            for (int tile = blockIdx.x; ok; tile += gridDim.x, ++it) {
                int m_tile, n_tile;
                if (!cursor.locate(tile, p, n_tiles, m_tile, n_tile)) break;
                const int buf = it & 1;
                const unsigned acc_phase = (it >> 1) & 1u;
                if (!mbar_wait(&tmem_empty[buf], acc_phase ^ 1u, abort)) break;
                tc_fence_after();
                const std::uint32_t acc = tmem_base + buf * kAccCols;
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!mbar_wait(&full_bar[stage], phase, abort)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    unsigned char* stage_base = tiles + stage * Plan::kStageBytes;
                    const std::uint64_t desc_a = make_smem_desc(stage_base);
                    // the B boxes are contiguous: 8-row groups stay 1024 bytes apart across the box boundary
                    const std::uint64_t desc_b = make_smem_desc(stage_base + Plan::kTileA);
#pragma unroll
                    for (int k = 0; k < kBlockKBytes / kUmmaKBytes; ++k) {
                        // 32 bytes further along K inside the swizzle atom: +2 in the address field
                        const std::uint64_t step = static_cast<std::uint64_t>(k * kUmmaKBytes) >> 4;
                        const std::uint32_t accumulate = (kb | k) != 0 ? 1u : 0u;
                        if (kFp8) umma_f8(acc, desc_a + step, desc_b + step, idesc, accumulate);
                        else umma_f16(acc, desc_a + step, desc_b + step, idesc, accumulate);
                    }
                    umma_commit(&empty_bar[stage]);  // the stage is free once these MMAs have read it
                    if (++stage == kStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (ok) umma_commit(&tmem_full[buf]);
            }
        }
    } else {
        // ===== epilogue: 4 warps, warp q owns TMEM lanes [32q, 32q+32) =====
        const int q = warp & 3;
        const ScatterTarget& sc = p.scatter;
        if (kScatter) {
            // every rank must have summed the previous call's rows before its landing area is overwritten
            if (lane < sc.num_ranks) {
                const auto* flag = reinterpret_cast<const std::uint64_t*>(sc.seg[sc.rank] + sc.done_off +
                                                                          static_cast<std::size_t>(lane) * sc.flag_stride);
                const std::uint64_t deadline = ptx::globaltimer_ns() + sc.timeout_ns;
                unsigned polls = 0;
                while (ptx::ld_acquire_sys(flag) + 1 < sc.epoch) {
                    if ((++polls & 63u) == 0 && (*abort || ptx::globaltimer_ns() > deadline)) {
                        if (!*abort) atomicCAS(&p.status[0], 0, 3);
                        *abort = 1;
                        break;
                    }
                    ptx::nanosleep(64);
                }
            }
            __syncwarp();
        }
        unsigned char* my_stage = staging + (q * 32 + lane) * kScatterRowPitch;
        TileCursor cursor;
        int it = 0;
        for (int tile = blockIdx.x;; tile += gridDim.x, ++it) {
            int m_tile, n_tile;
            if (!cursor.locate(tile, p, n_tiles, m_tile, n_tile)) break;
            const int buf = it & 1;
            const unsigned acc_phase = (it >> 1) & 1u;
            if (!mbar_wait(&tmem_full[buf], acc_phase, abort)) break;
            tc_fence_after();
            const int row = m_tile * kBlockM + q * 32 + lane;
            const bool valid = row < p.expert_counts[cursor.expert];
            const long long out_row = static_cast<long long>(p.expert_offsets[cursor.expert]) + row;
            __nv_bfloat16* out = p.out + out_row * p.n + n_tile * kOutN;
            // FP8: the per-row activation scale and the per-output-channel weight scale factor out of the K sum
            const float a_scale = (kFp8 && valid) ? p.a_scales[out_row] : 1.0f;
            const float* w_scale = kFp8 ? p.w_scales + static_cast<long long>(cursor.expert) * w_rows_per_expert + n_tile * kOutN : nullptr;
            const std::uint32_t lane_base = tmem_base + (static_cast<std::uint32_t>(q * 32) << 16) + buf * kAccCols;
            if (kScatter) {
                int owner = -1, token = 0, slot = -1;
                float weight = 1.0f;
                if (valid) {
                    const long long* meta = sc.source_meta + out_row * 3;
                    owner = static_cast<int>(meta[0]);
                    token = static_cast<int>(meta[1]);
                    slot = static_cast<int>(meta[2]);
                    if (sc.row_weights != nullptr) weight = sc.row_weights[out_row];
                }
                const bool send = valid && owner >= 0 && owner < sc.num_ranks && slot >= 0 && slot < sc.num_topk && token >= 0;
                unsigned char* dst = nullptr;
                if (send)
                    dst = sc.seg[owner] + sc.stage_off +
                          (static_cast<std::size_t>(token) * sc.num_topk + slot) * static_cast<std::size_t>(sc.row_stride) +
                          static_cast<std::size_t>(n_tile) * kOutN * 2;
                const unsigned long long dst_bits = reinterpret_cast<unsigned long long>(dst);
                const unsigned char* warp_stage = staging + q * 32 * kScatterRowPitch;
                const int sub = lane & 15;  // 16-byte piece of a 256-byte row segment
#pragma unroll 1
                for (int half = 0; half < kOutN / kBlockN; ++half) {
                    // (1) lane = row: accumulator columns -> weighted BF16 -> this lane's staging row
#pragma unroll 1
                    for (int c0 = 0; c0 < kBlockN; c0 += 32) {
                        std::uint32_t g[32];
                        tmem_ld_32x32(lane_base + half * kBlockN + c0, g);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 32; i += 8) {
                            uint4 packed;
                            __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
                            for (int j = 0; j < 4; ++j)
                                h[j] = __floats2bfloat162_rn(__uint_as_float(g[i + 2 * j]) * weight, __uint_as_float(g[i + 2 * j + 1]) * weight);
                            *reinterpret_cast<uint4*>(my_stage + (c0 + i) * 2) = packed;
                        }
                    }
                    if (half == kOutN / kBlockN - 1) {
                        // the accumulator has been read completely: the MMA warp may start the tile after next
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&tmem_empty[buf]);
                    } else {
                        __syncwarp();
                    }
                    // (2) half a warp = one row: 16 lanes store 256 contiguous bytes into the owner's slot, so a
                    //     peer receives full 128-byte write packets instead of 32 scattered 16-byte pieces
#pragma unroll 4
                    for (int r = 0; r < 32; r += 2) {
                        const int row_lane = r + (lane >> 4);
                        const unsigned long long to = __shfl_sync(0xffffffffu, dst_bits, row_lane);
                        const uint4 v = *reinterpret_cast<const uint4*>(warp_stage + row_lane * kScatterRowPitch + sub * 16);
                        if (to != 0ull) ptx::st_v4(reinterpret_cast<unsigned char*>(to) + half * kBlockN * 2 + sub * 16, v);
                    }
                    __syncwarp();  // the staging rows are rewritten by the next half / tile
                }
                continue;
            }
#pragma unroll 1
            for (int c0 = 0; c0 < kOutN; c0 += 32) {
                std::uint32_t g[32];
                tmem_ld_32x32(lane_base + c0, g);
                float v[32];
                if (kSwiGLU) {
                    std::uint32_t u[32];
                    tmem_ld_32x32(lane_base + kBlockN + c0, u);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        float gate = __uint_as_float(g[i]);
                        float up = __uint_as_float(u[i]);
                        if (kFp8) {
                            gate *= a_scale * __ldg(w_scale + c0 + i);
                            up *= a_scale * __ldg(w_scale + p.n + c0 + i);
                        }
                        v[i] = gate / (1.0f + __expf(-gate)) * up;
                    }
                } else {
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        v[i] = __uint_as_float(g[i]);
                        if (kFp8) v[i] *= a_scale * __ldg(w_scale + c0 + i);
                    }
                }
                if (valid) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        uint4 packed;
                        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
                        for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(v[i + 2 * j], v[i + 2 * j + 1]);
                        *reinterpret_cast<uint4*>(out + c0 + i) = packed;
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&tmem_empty[buf]);
        }
        if (kScatter) ptx::fence_sys();  // this thread's rows before the CTA is counted as finished
    }

    // ---- teardown: every role has left its loop (normally or through the abort latch)
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
    if (threadIdx.x == 0 && *abort) atomicCAS(&p.status[0], 0, 1);
    if (kScatter && threadIdx.x == 0) {
        const ScatterTarget& sc = p.scatter;
        ptx::fence_sys();
        const unsigned long long finished = atomicAdd(sc.cta_done, 1ull) + 1ull;
        if (finished == gridDim.x) {
            // last CTA of this launch: all rows of all CTAs are written; tell every owner (unless something gave up).
            // Launches that share the counter are stream-ordered, so the next one finds it at zero again.
            *sc.cta_done = 0ull;
            ptx::fence_sys();
            if (*reinterpret_cast<volatile int*>(p.status) == 0) {
                for (int r = 0; r < sc.num_ranks; ++r)
                    ptx::st_release_sys(reinterpret_cast<std::uint64_t*>(sc.seg[r] + sc.sig_off + static_cast<std::size_t>(sc.rank) * sc.flag_stride),
                                        sc.epoch);
            }
        }
    }
}

// ---- host side ----------------------------------------------------------------------------------

namespace {

using EncodeTiled = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                 const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encode_tiled() {
    static EncodeTiled fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* entry = nullptr;
        cudaDriverEntryPointQueryResult result;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &entry, cudaEnableDefault, &result) == cudaSuccess &&
            result == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiled>(entry);
    });
    return fn;
}

// [rows, k] row-major (bf16 or 1-byte fp8), box = 128 bytes of K x box_rows rows, 128-byte swizzle
bool make_map(CUtensorMap* map, const void* base, std::uint64_t rows, std::uint64_t k, std::uint32_t box_rows, bool fp8) {
    EncodeTiled encode = encode_tiled();
    if (encode == nullptr) return false;
    const std::uint64_t elem_bytes = fp8 ? 1 : 2;
    const cuuint64_t dims[2] = {k, rows};
    const cuuint64_t strides[1] = {k * elem_bytes};
    const cuuint32_t box[2] = {static_cast<cuuint32_t>(kBlockKBytes / elem_bytes), box_rows};
    const cuuint32_t elem[2] = {1, 1};
    return encode(map, fp8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <bool kSwiGLU, bool kFp8, int kBoxesB, bool kScatter = false>
cudaError_t launch(const CUtensorMap& map_a, const CUtensorMap& map_b, const GroupedGemmParams& p, int ctas, cudaStream_t stream) {
    static bool configured[64] = {false};
    int device = 0;
    cudaError_t status = cudaGetDevice(&device);
    if (status != cudaSuccess) return status;
    // the scatter variant adds its staging rows and keeps 512 bytes of alignment slack (checked in the kernel)
    constexpr int smem = kScatter ? SmemPlan<kBoxesB>::kStages * SmemPlan<kBoxesB>::kStageBytes + 256 + kScatterStagingBytes + 512
                                  : SmemPlan<kBoxesB>::kBytes;
    if (device >= 0 && device < 64 && !configured[device]) {
        status = cudaFuncSetAttribute(grouped_gemm_kernel<kSwiGLU, kFp8, kBoxesB, kScatter>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (status != cudaSuccess) return status;
        configured[device] = true;
    }
    grouped_gemm_kernel<kSwiGLU, kFp8, kBoxesB, kScatter><<<ctas, kThreads, smem, stream>>>(map_a, map_b, p);
    return cudaGetLastError();
}

}  // namespace

}  // namespace gemm

namespace {
const char* run_grouped_gemm(const void* a, const void* w, void* out, const float* a_scales, const float* w_scales,
                             const int* expert_offsets, const int* expert_counts, int* status, int rows_capacity,
                             int num_experts, int n, int k, bool swiglu, bool fp8, const gemm::ScatterTarget* target,
                             cudaStream_t stream) {
    using namespace gemm;
    const int block_k = kBlockKBytes / (fp8 ? 1 : 2);
    if (n % kBlockN != 0 || k % block_k != 0 || n <= 0 || k <= 0)
        return "n must be a multiple of 128 and k a multiple of 64 (bf16) / 128 (fp8)";
    if (reinterpret_cast<std::uintptr_t>(a) % 16 || reinterpret_cast<std::uintptr_t>(w) % 16 ||
        reinterpret_cast<std::uintptr_t>(out) % 16)
        return "operands must be 16-byte aligned";
    if (target != nullptr) {
        if (swiglu || fp8 || n % (2 * kBlockN) != 0) return "the scatter epilogue needs a plain BF16 GEMM with n a multiple of 256";
        if (target->num_ranks < 1 || target->num_ranks > kScatterMaxRanks || target->rank < 0 || target->rank >= target->num_ranks)
            return "scatter target: bad rank table";
        if (target->row_stride % 16 != 0 || target->row_stride < 2 * n || target->stage_off % 16 != 0 || target->epoch == 0 ||
            target->cta_done == nullptr || target->source_meta == nullptr)
            return "scatter target: bad landing-area description";
    }
    if (fp8 && (a_scales == nullptr || w_scales == nullptr)) return "fp8 operands need their scales";
    CUtensorMap map_a, map_b;
    const std::uint64_t w_rows = static_cast<std::uint64_t>(num_experts) * (swiglu ? 2 : 1) * n;
    if (!make_map(&map_a, a, static_cast<std::uint64_t>(rows_capacity), static_cast<std::uint64_t>(k), kBlockM, fp8) ||
        !make_map(&map_b, w, w_rows, static_cast<std::uint64_t>(k), kBlockN, fp8))
        return "cuTensorMapEncodeTiled failed";
    GroupedGemmParams p{};
    p.expert_offsets = expert_offsets;
    p.expert_counts = expert_counts;
    p.out = static_cast<__nv_bfloat16*>(out);
    p.a_scales = a_scales;
    p.w_scales = w_scales;
    p.status = status;
    p.num_experts = num_experts;
    p.n = n;
    p.k = k;
    p.rows_capacity = rows_capacity;
    if (target != nullptr) p.scatter = *target;
    int device = 0, sms = 0;
    if (cudaGetDevice(&device) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess)
        return "cannot query the device";
    cudaError_t err;
    const bool wide = n % (2 * kBlockN) == 0;  // plain GEMM: 256-column tiles whenever n allows
    if (target != nullptr) {
        err = launch<false, false, 2, true>(map_a, map_b, p, sms, stream);
    } else if (fp8) {
        err = swiglu ? launch<true, true, 2>(map_a, map_b, p, sms, stream)
              : wide ? launch<false, true, 2>(map_a, map_b, p, sms, stream)
                     : launch<false, true, 1>(map_a, map_b, p, sms, stream);
    } else {
        err = swiglu ? launch<true, false, 2>(map_a, map_b, p, sms, stream)
              : wide ? launch<false, false, 2>(map_a, map_b, p, sms, stream)
                     : launch<false, false, 1>(map_a, map_b, p, sms, stream);
    }
    return err == cudaSuccess ? nullptr : cudaGetErrorString(err);
}
}  // namespace

const char* grouped_gemm(const void* a, const void* w, void* out, const float* a_scales, const float* w_scales,
                         const int* expert_offsets, const int* expert_counts, int* status, int rows_capacity,
                         int num_experts, int n, int k, bool swiglu, bool fp8, cudaStream_t stream) {
    return run_grouped_gemm(a, w, out, a_scales, w_scales, expert_offsets, expert_counts, status, rows_capacity, num_experts,
                            n, k, swiglu, fp8, nullptr, stream);
}

const char* grouped_gemm_scatter(const void* a, const void* w, const int* expert_offsets, const int* expert_counts,
                                 int* status, int rows_capacity, int num_experts, int n, int k,
                                 const gemm::ScatterTarget& target, cudaStream_t stream) {
    // `out` is never written by the scatter epilogue; the A pointer stands in to satisfy the alignment check
    return run_grouped_gemm(a, w, const_cast<void*>(a), nullptr, nullptr, expert_offsets, expert_counts, status, rows_capacity,
                            num_experts, n, k, false, false, &target, stream);
}

int grouped_gemm_ctas() {
    int device = 0, sms = 0;
    if (cudaGetDevice(&device) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess)
        return 0;
    return sms;
}

}  // namespace bep
