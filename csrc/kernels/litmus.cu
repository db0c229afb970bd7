// READY/ACK publication litmus over peer-visible memory: the smallest program that exercises the
// memory-model rules the transport relies on (parity: the reference's mapped-host-memory litmus,
// tests/mapped_litmus.cu:101-193, here for HBM reached over NVLink).  Two publication chains:
//   method 0  payload by ordinary stores, then `st.release.sys` of a flag written by exactly one side;
//             `ld.acquire.sys` on the other side, then plain loads of the payload;
//   method 1  the chain of the dispatch send warps: payload staged in shared memory and pushed with
//             `cp.async.bulk` by lane 31, `cp.async.bulk.wait_group 0` and `fence.acq_rel.sys` on that lane,
//             `__syncwarp()`, then `st.relaxed.sys` of the flag by lane 0; the other side reads the flag
//             with `ld.acquire.sys`, issues `fence.proxy.async` and fetches the payload with a bulk load.
//             (Without the fence the same chain passed here on two GPUs a million times and still let a flag
//             overtake part of a 14 KB row on four: a passing litmus is no proof of the rule.)
// An ACK flag goes the other way in both.
//
// role 0 = producer, role 1 = consumer, role -1 = both roles as two CTAs of one cooperative launch on
// one GPU (the only legal way to run two mutually waiting parties on a single device).
// Every wait is bounded; on expiry status[0] = 1 and the kernel returns.
//
// Memory of each side (at least 256 + 8 * words bytes, zero-initialised):
//   +0   u64 ready   (written by the producer into the consumer's memory)
//   +128 u64 ack     (written by the consumer into the producer's memory)
//   +256 payload words
#include "litmus.hpp"

#include <cstdint>

#include "ptx.cuh"

namespace bep {

namespace {

__device__ __forceinline__ unsigned long long mix(unsigned long long round, unsigned long long k) {
    unsigned long long v = (round + 1) * 0x9E3779B97F4A7C15ull + k * 0xC2B2AE3D27D4EB4Full;
    v ^= v >> 29;
    return v * 0xBF58476D1CE4E5B9ull;
}

__device__ bool wait_for(const std::uint64_t* flag, std::uint64_t value, unsigned long long deadline) {
    while (ptx::ld_acquire_sys(flag) != value) {
        if (ptx::globaltimer_ns() > deadline) return false;
    }
    return true;
}

constexpr int kLitmusMaxBulkWords = 2048;

__global__ void litmus_kernel(std::uint8_t* mine, std::uint8_t* theirs, int role, int rounds, int words,
                              long long* status, unsigned long long timeout_ns, int method) {
    __shared__ __align__(128) unsigned long long stage[kLitmusMaxBulkWords];
    __shared__ __align__(8) unsigned long long bar;
    // role -1: CTA 0 is the producer living in `mine`, CTA 1 the consumer living in `theirs`
    std::uint8_t* own = mine;
    std::uint8_t* peer = theirs;
    int my_role = role;
    if (role < 0) {
        my_role = blockIdx.x;
        if (my_role == 1) {
            own = theirs;
            peer = mine;
        }
    }
    const unsigned lane = threadIdx.x;
    if (method == 1 && lane == 0) {
        ptx::mbar_init(reinterpret_cast<std::uint64_t*>(&bar), 1);
        ptx::mbar_fence_init();
    }
    __syncwarp();
    unsigned parity = 0;
    const unsigned long long start = ptx::globaltimer_ns();
    const unsigned long long deadline = start + timeout_ns;
    long long mismatches = 0;
    int done = 0;
    bool ok = true;
    for (int r = 0; r < rounds && ok; ++r) {
        if (my_role == 0 && method == 1) {
            for (int k = lane; k < words; k += 32) stage[k] = mix(r, k);
            ptx::fence_proxy_async_smem();
            __syncwarp();
            if (lane == 31) {
                ptx::bulk_s2g(peer + 256, stage, static_cast<unsigned>(words) * 8u);
                ptx::bulk_commit();
                ptx::bulk_wait_all();
                ptx::fence_sys();
            }
            __syncwarp();
            if (lane == 0) {
                ptx::st_relaxed_sys(reinterpret_cast<std::uint64_t*>(peer), static_cast<std::uint64_t>(r + 1));
                ok = wait_for(reinterpret_cast<const std::uint64_t*>(own + 128), static_cast<std::uint64_t>(r + 1), deadline);
            }
        } else if (my_role == 0) {
            auto* payload = reinterpret_cast<unsigned long long*>(peer + 256);
            for (int k = lane; k < words; k += 32) payload[k] = mix(r, k);
            __syncwarp();
            if (lane == 0) {
                ptx::st_release_sys(reinterpret_cast<std::uint64_t*>(peer), static_cast<std::uint64_t>(r + 1));
                ok = wait_for(reinterpret_cast<const std::uint64_t*>(own + 128), static_cast<std::uint64_t>(r + 1), deadline);
            }
        } else {
            if (lane == 0) ok = wait_for(reinterpret_cast<const std::uint64_t*>(own), static_cast<std::uint64_t>(r + 1), deadline);
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            if (ok && method == 1) {
                ptx::fence_proxy_async();
                if (lane == 0) {
                    ptx::mbar_expect_tx(reinterpret_cast<std::uint64_t*>(&bar), static_cast<unsigned>(words) * 8u);
                    ptx::bulk_g2s(stage, own + 256, static_cast<unsigned>(words) * 8u, reinterpret_cast<std::uint64_t*>(&bar));
                }
                bool landed = true;
                while (!ptx::mbar_try_wait(reinterpret_cast<std::uint64_t*>(&bar), parity)) {
                    if (ptx::globaltimer_ns() > deadline) {
                        landed = false;
                        break;
                    }
                }
                parity ^= 1u;
                ok = __all_sync(0xffffffffu, landed) != 0;
                if (ok) {
                    for (int k = lane; k < words; k += 32)
                        if (stage[k] != mix(r, k)) ++mismatches;
                    __syncwarp();
                    if (lane == 0) ptx::st_relaxed_sys(reinterpret_cast<std::uint64_t*>(peer + 128), static_cast<std::uint64_t>(r + 1));
                }
            } else if (ok) {
                const auto* payload = reinterpret_cast<const volatile unsigned long long*>(own + 256);
                for (int k = lane; k < words; k += 32)
                    if (payload[k] != mix(r, k)) ++mismatches;
                __syncwarp();
                if (lane == 0) ptx::st_release_sys(reinterpret_cast<std::uint64_t*>(peer + 128), static_cast<std::uint64_t>(r + 1));
            }
        }
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        if (ok) ++done;
    }
    for (int o = 16; o > 0; o >>= 1) mismatches += __shfl_xor_sync(0xffffffffu, mismatches, o);
    if (lane == 0) {
        long long* out = status + (role < 0 ? my_role * 4 : 0);
        out[0] = ok ? 0 : 1;
        out[1] = mismatches;
        out[2] = done;
        out[3] = static_cast<long long>(ptx::globaltimer_ns() - start);
    }
}

}  // namespace

const char* litmus_pingpong(void* mine, void* theirs, int role, int rounds, int words, long long* status,
                            unsigned long long timeout_ns, cudaStream_t stream, int method) {
    if (role < -1 || role > 1 || rounds < 1 || words < 0 || method < 0 || method > 1) return "bad litmus arguments";
    if (method == 1 && (words < 2 || words % 2 != 0 || words > kLitmusMaxBulkWords))
        return "the bulk-copy litmus needs an even number of payload words, at most 2048";
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(role < 0 ? 2 : 1, 1, 1);
    config.blockDim = dim3(32, 1, 1);
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeCooperative;  // both CTAs resident when they wait for each other
    attribute[0].val.cooperative = 1;
    config.attrs = attribute;
    config.numAttrs = 1;
    const cudaError_t err = cudaLaunchKernelEx(&config, litmus_kernel, static_cast<std::uint8_t*>(mine),
                                               static_cast<std::uint8_t*>(theirs), role, rounds, words, status, timeout_ns, method);
    return err == cudaSuccess ? nullptr : cudaGetErrorString(err);
}

}  // namespace bep
