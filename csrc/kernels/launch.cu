// The CUDA translation unit: every __global__ kernel of the library and its launch wrapper.
#include "launch.hpp"

#include <algorithm>
#include <mutex>

#include "combine.cuh"
#include "dispatch.cuh"
#include "combine_push.cuh"
#include "fused_reduce.cuh"

namespace bep {

std::size_t dispatch_shared_bytes(const SegmentLayout& lay, int tx_warps, int rx_warps, bool use_tma, int stages,
                                  int send_ctas) {
    return dispatch_smem_bytes(lay, tx_warps, rx_warps, use_tma, stages, send_ctas);
}

bool role_profiling_enabled() { return BEP_ENABLE_PROFILING != 0; }

cudaError_t configure_kernels(std::size_t dispatch_smem) {
    // One attribute per kernel per process: several buffers may be alive, so only ever raise it.
    static std::mutex mutex;
    static std::size_t current[64] = {0};
    std::lock_guard<std::mutex> guard(mutex);
    int device = 0;
    cudaError_t status = cudaGetDevice(&device);
    if (status != cudaSuccess) return status;
    if (device < 0 || device >= 64) return cudaErrorInvalidDevice;
    if (dispatch_smem > current[device]) {
        status = cudaFuncSetAttribute(dispatch_kernel<kSmallCtaThreads>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      static_cast<int>(dispatch_smem));
        if (status != cudaSuccess) return status;
        status = cudaFuncSetAttribute(dispatch_kernel<kMaxWarps * 32>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      static_cast<int>(dispatch_smem));
        if (status != cudaSuccess) return status;
        current[device] = dispatch_smem;
    }
    return cudaSuccess;
}

int dispatch_resident_ctas(int threads, std::size_t smem) {
    int per_sm = 0, device = 0, sms = 0;
    if (cudaGetDevice(&device) != cudaSuccess) return 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return 0;
    const cudaError_t status = threads <= kSmallCtaThreads
                                   ? cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, dispatch_kernel<kSmallCtaThreads>, threads, smem)
                                   : cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, dispatch_kernel<kMaxWarps * 32>, threads, smem);
    if (status != cudaSuccess) return 0;
    return per_sm * sms;
}

int combine_resident_ctas(int threads) {
    int per_sm = 0, device = 0, sms = 0;
    if (cudaGetDevice(&device) != cudaSuccess) return 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, combine_kernel, threads, 0) != cudaSuccess) return 0;
    return per_sm * sms;
}

namespace {

template <typename Kernel, typename Args>
cudaError_t cooperative_launch(Kernel kernel, const Args& args, dim3 grid, int threads, std::size_t smem,
                               cudaStream_t stream) {
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = dim3(static_cast<unsigned>(threads), 1, 1);
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeCooperative;  // every CTA resident: the waits inside are safe
    attribute[0].val.cooperative = 1;
    config.attrs = attribute;
    config.numAttrs = 1;
    return cudaLaunchKernelEx(&config, kernel, args);
}

}  // namespace

cudaError_t launch_dispatch(const DispatchLaunch& launch, int ctas, int threads, std::size_t smem,
                            cudaStream_t stream) {
    const dim3 grid(ctas, launch.num_virtual, 1);
    if (threads <= kSmallCtaThreads) return cooperative_launch(dispatch_kernel<kSmallCtaThreads>, launch, grid, threads, smem, stream);
    return cooperative_launch(dispatch_kernel<kMaxWarps * 32>, launch, grid, threads, smem, stream);
}

cudaError_t launch_combine(const CombineLaunch& launch, int channels, std::size_t crow_stride, cudaStream_t stream) {
    const std::size_t smem = static_cast<std::size_t>(kCombineWarps) * crow_stride;
    static std::mutex mutex;
    static std::size_t configured[64] = {0};
    {
        std::lock_guard<std::mutex> guard(mutex);
        int device = 0;
        cudaError_t status = cudaGetDevice(&device);
        if (status != cudaSuccess) return status;
        if (device >= 0 && device < 64 && smem > configured[device]) {
            status = cudaFuncSetAttribute(combine_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
            if (status != cudaSuccess) return status;
            configured[device] = smem;
        }
    }
    return cooperative_launch(combine_kernel, launch, dim3(channels, launch.num_virtual, 1), kCombineWarps * 32, smem, stream);
}

cudaError_t launch_combine_push(const CombinePushArgs& args, int reduce_ctas, std::size_t smem, cudaStream_t stream) {
    static std::mutex mutex;
    static std::size_t configured[64] = {0};
    {
        std::lock_guard<std::mutex> guard(mutex);
        int device = 0;
        cudaError_t status = cudaGetDevice(&device);
        if (status != cudaSuccess) return status;
        if (device >= 0 && device < 64 && smem > configured[device]) {
            status = cudaFuncSetAttribute(combine_push_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
            if (status != cudaSuccess) return status;
            configured[device] = smem;
        }
    }
    combine_push_kernel<<<args.forward_ctas + reduce_ctas, kFusedReduceThreads, smem, stream>>>(args);
    return cudaGetLastError();
}

cudaError_t launch_fused_reduce(const FusedReduceArgs& args, int ctas, cudaStream_t stream) {
    switch (fused_reduce_groups(args.slots)) {
        case 4: fused_reduce_kernel<4><<<ctas, kFusedReduceThreads, 0, stream>>>(args); break;
        case 2: fused_reduce_kernel<2><<<ctas, kFusedReduceThreads, 0, stream>>>(args); break;
        default: fused_reduce_kernel<1><<<ctas, kFusedReduceThreads, 0, stream>>>(args); break;
    }
    return cudaGetLastError();
}

}  // namespace bep
