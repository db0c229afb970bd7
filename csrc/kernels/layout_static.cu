// bep_route_layout_static: the dispatch kernel's routing-layout phase as a stand-alone entry point
// whose cross-CTA scratch lives in a file-scope __device__ array.  See layout_static.h for the
// contract.  Nothing in this file allocates: no cudaMalloc/cudaFree, no PyTorch tensors.
#include "layout_static.h"

#include <mutex>

#include <cuda_runtime.h>

namespace {

constexpr int kThreads = 256;
constexpr unsigned long long kBarrierTimeoutNs = 2000000000ull;

struct StaticScratch {
    unsigned long long barrier;  // arrivals of the one grid barrier; cleared before every launch
    unsigned long long reserved[31];
    int hist[BEP_STATIC_MAX_CHANNELS * (BEP_STATIC_MAX_EXPERTS + BEP_STATIC_MAX_RANKS)];
};

// The scratch itself.  In host code this name is only a handle for cudaGetSymbolAddress; the kernel
// gets the real device address as an argument.
static __device__ __align__(256) unsigned char g_layout_scratch[sizeof(StaticScratch)];

__device__ __forceinline__ unsigned long long now_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__global__ void __launch_bounds__(kThreads, 1)
route_layout_static_kernel(StaticScratch* scratch, const long long* __restrict__ topk_idx, int T, int K, int E, int P,
                           unsigned* plan_mask, int* plan_slot, int* plan_expert_ord, int* plan_counts, int* status) {
    __shared__ int cnt_e[BEP_STATIC_MAX_EXPERTS];
    __shared__ unsigned bits_e[BEP_STATIC_MAX_EXPERTS];
    __shared__ int total_e[BEP_STATIC_MAX_EXPERTS];
    __shared__ int cnt_r[BEP_STATIC_MAX_RANKS];
    __shared__ unsigned bits_r[BEP_STATIC_MAX_RANKS];
    __shared__ int total_r[BEP_STATIC_MAX_RANKS];
    __shared__ int barrier_failed;

    const int C = gridDim.x, c = blockIdx.x;
    const int El = E / P;
    const int Tc = (T + C - 1) / C;
    const int t0 = min(T, c * Tc), t1 = min(T, t0 + Tc);
    const unsigned lane = threadIdx.x & 31u;
    const unsigned lt_mask = (1u << lane) - 1u;

    for (int i = threadIdx.x; i < E; i += blockDim.x) {
        cnt_e[i] = 0;
        bits_e[i] = 0;
    }
    if (threadIdx.x < BEP_STATIC_MAX_RANKS) {
        cnt_r[threadIdx.x] = 0;
        bits_r[threadIdx.x] = 0;
    }
    if (threadIdx.x == 0) barrier_failed = 0;
    __syncthreads();
    // per-channel histograms + route validation
    for (int t = t0 + threadIdx.x; t < t1; t += blockDim.x) {
        unsigned mask = 0;
        const long long* row = topk_idx + static_cast<size_t>(t) * K;
        for (int k = 0; k < K; ++k) {
            const long long e = row[k];
            if (e == -1) continue;
            bool bad = e < -1 || e >= E;
            for (int k2 = 0; k2 < k && !bad; ++k2) bad = row[k2] == e;
            if (bad) {
                if (atomicCAS(&status[0], 0, 2) == 0) {
                    status[1] = t;
                    status[2] = k;
                }
                continue;
            }
            mask |= 1u << static_cast<int>(e / El);
            atomicAdd(&cnt_e[e], 1);
        }
        plan_mask[t] = mask;
        for (unsigned m = mask; m; m &= m - 1) atomicAdd(&cnt_r[__ffs(m) - 1], 1);
    }
    __syncthreads();
    int* hist = scratch->hist + static_cast<size_t>(c) * (E + P);
    for (int i = threadIdx.x; i < E + P; i += blockDim.x) hist[i] = i < E ? cnt_e[i] : cnt_r[i - E];
    // grid barrier (cooperative launch: every CTA is resident); bounded
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        atomicAdd(&scratch->barrier, 1ull);
        const unsigned long long deadline = now_ns() + kBarrierTimeoutNs;
        while (*reinterpret_cast<volatile unsigned long long*>(&scratch->barrier) < static_cast<unsigned long long>(C)) {
            if (now_ns() > deadline) {
                atomicCAS(&status[0], 0, 21);
                barrier_failed = 1;
                break;
            }
            __nanosleep(64);
        }
        __threadfence();
    }
    __syncthreads();
    if (barrier_failed) return;
    // exclusive prefix over earlier channels
    for (int i = threadIdx.x; i < E + P; i += blockDim.x) {
        int base = 0, total = 0;
        for (int c2 = 0; c2 < C; ++c2) {
            const int v = __ldcg(scratch->hist + static_cast<size_t>(c2) * (E + P) + i);
            total += v;
            if (c2 < c) base += v;
        }
        if (i < E) {
            cnt_e[i] = base;
            total_e[i] = total;
        } else {
            cnt_r[i - E] = 0;
            total_r[i - E] = total;
        }
    }
    __syncthreads();
    if (c == 0) {
        for (int i = threadIdx.x; i < P + E; i += blockDim.x) plan_counts[i] = i < P ? total_r[i] : total_e[i - P];
        for (int i = threadIdx.x; i < C * P; i += blockDim.x)
            plan_counts[P + E + i] = __ldcg(scratch->hist + static_cast<size_t>(i / P) * (E + P) + E + i % P);
    }
    if (threadIdx.x < 32) {
        // stable ordinals, 32 tokens at a time (lane = token)
        for (int base_t = t0; base_t < t1; base_t += 32) {
            const int t = base_t + lane;
            const bool active = t < t1;
            const unsigned mask = active ? plan_mask[t] : 0u;
            const long long* row = topk_idx + static_cast<size_t>(active ? t : 0) * K;
            for (int k = 0; k < K; ++k) {
                const long long e = active ? row[k] : -1;
                if (e >= 0 && e < E) atomicOr(&bits_e[e], 1u << lane);
            }
            for (unsigned m = mask; m; m &= m - 1) atomicOr(&bits_r[__ffs(m) - 1], 1u << lane);
            __syncwarp();
            if (active) {
                for (int k = 0; k < K; ++k) {
                    const long long e = row[k];
                    plan_expert_ord[static_cast<size_t>(t) * K + k] =
                        (e >= 0 && e < E) ? cnt_e[e] + __popc(bits_e[e] & lt_mask) : -1;
                }
                for (int d = 0; d < P; ++d)
                    plan_slot[static_cast<size_t>(t) * P + d] =
                        (mask >> d & 1u) ? cnt_r[d] + __popc(bits_r[d] & lt_mask) : -1;
            }
            __syncwarp();
            for (int k = 0; k < K; ++k) {
                const long long e = active ? row[k] : -1;
                if (e >= 0 && e < E) {
                    const unsigned b = bits_e[e];
                    if (lane == 31u - __clz(b)) cnt_e[e] += __popc(b);
                }
            }
            for (unsigned m = mask; m; m &= m - 1) {
                const int d = __ffs(m) - 1;
                const unsigned b = bits_r[d];
                if (lane == 31u - __clz(b)) cnt_r[d] += __popc(b);
            }
            __syncwarp();
            for (int k = 0; k < K; ++k) {
                const long long e = active ? row[k] : -1;
                if (e >= 0 && e < E) bits_e[e] = 0;
            }
            for (unsigned m = mask; m; m &= m - 1) bits_r[__ffs(m) - 1] = 0;
            __syncwarp();
        }
    }
}

struct DeviceSetup {
    bool ready = false;
    StaticScratch* scratch = nullptr;
    int resident_ctas = 0;
};

// One-time set-up per device: device address of the scratch array and how many CTAs fit at once.
cudaError_t device_setup(int device, DeviceSetup** out) {
    static std::mutex mutex;
    static DeviceSetup setups[64];
    if (device < 0 || device >= 64) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> guard(mutex);
    DeviceSetup& s = setups[device];
    if (!s.ready) {
        void* address = nullptr;
        cudaError_t status = cudaGetSymbolAddress(&address, g_layout_scratch);  // `device` is current
        if (status != cudaSuccess) return status;
        int per_sm = 0, sms = 0;
        status = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, route_layout_static_kernel, kThreads, 0);
        if (status != cudaSuccess) return status;
        status = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
        if (status != cudaSuccess) return status;
        s.scratch = static_cast<StaticScratch*>(address);
        s.resident_ctas = per_sm * sms;
        s.ready = true;
    }
    *out = &s;
    return cudaSuccess;
}

}  // namespace

extern "C" unsigned long long bep_route_layout_static_scratch_bytes(void) { return sizeof(StaticScratch); }

extern "C" int bep_route_layout_static(const int64_t* topk_idx, int num_tokens, int num_topk, int num_experts,
                                       int num_ranks, int num_channels, uint32_t* plan_mask, int* plan_slot,
                                       int* plan_expert_ord, int* plan_counts, int* status, cudaStream_t stream) {
    if (num_channels > BEP_STATIC_MAX_CHANNELS || num_experts > BEP_STATIC_MAX_EXPERTS ||
        num_ranks > BEP_STATIC_MAX_RANKS || num_topk > BEP_STATIC_MAX_TOPK)
        return BEP_STATIC_ERR_TOO_LARGE;
    if (num_tokens < 0 || num_topk < 1 || num_experts < 1 || num_ranks < 1 || num_channels < 1 ||
        num_experts % num_ranks != 0 || plan_counts == nullptr || status == nullptr ||
        (num_tokens > 0 && (topk_idx == nullptr || plan_mask == nullptr || plan_slot == nullptr || plan_expert_ord == nullptr)))
        return BEP_STATIC_ERR_ARGUMENT;
    int device = 0;
    cudaError_t err = cudaGetDevice(&device);
    if (err != cudaSuccess) return static_cast<int>(err);
    DeviceSetup* setup = nullptr;
    err = device_setup(device, &setup);
    if (err != cudaSuccess) return static_cast<int>(err);
    if (num_channels > setup->resident_ctas) return BEP_STATIC_ERR_RESIDENCY;

    // The array keeps whatever the previous call left: the barrier counter must start at zero.
    // (The histograms need no clearing: every word that is read was written by this launch.)
    err = cudaMemsetAsync(&setup->scratch->barrier, 0, sizeof(unsigned long long), stream);
    if (err != cudaSuccess) return static_cast<int>(err);
    err = cudaMemsetAsync(status, 0, 4 * sizeof(int), stream);
    if (err != cudaSuccess) return static_cast<int>(err);

    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(static_cast<unsigned>(num_channels), 1, 1);
    config.blockDim = dim3(kThreads, 1, 1);
    config.dynamicSmemBytes = 0;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeCooperative;
    attribute[0].val.cooperative = 1;
    config.attrs = attribute;
    config.numAttrs = 1;
    err = cudaLaunchKernelEx(&config, route_layout_static_kernel, setup->scratch,
                             reinterpret_cast<const long long*>(topk_idx), num_tokens, num_topk, num_experts, num_ranks,
                             plan_mask, plan_slot, plan_expert_ord, plan_counts, status);
    return static_cast<int>(err);
}
