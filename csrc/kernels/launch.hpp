// Host-callable entry points of the CUDA translation unit (csrc/kernels/launch.cu).  The runtime
// (plain C++, built without nvcc) only sees these.
#pragma once

#include <cstddef>

#include <cuda_runtime.h>

#include "combine_push.cuh"
#include "fused_reduce.cuh"
#include "protocol.cuh"

namespace bep {

// Shared-memory bytes the dispatch kernel needs for this configuration (`stages` row buffers per send warp).
std::size_t dispatch_shared_bytes(const SegmentLayout& lay, int tx_warps, int rx_warps, bool use_tma, int stages,
                                  int send_ctas);

// Raise (never lower) the kernels' dynamic shared-memory limit; thread-safe, idempotent.
cudaError_t configure_kernels(std::size_t dispatch_smem_bytes);

// How many CTAs of `threads` threads and `smem` dynamic bytes fit on the current device at once.
int dispatch_resident_ctas(int threads, std::size_t smem);
int combine_resident_ctas(int threads);

// Cooperative launches: grid = (CTAs per rank, virtual ranks); dispatch: channels + dedicated sender CTAs.
cudaError_t launch_dispatch(const DispatchLaunch& launch, int ctas, int threads, std::size_t smem,
                            cudaStream_t stream);
cudaError_t launch_combine(const CombineLaunch& launch, int channels, std::size_t crow_stride, cudaStream_t stream);

// Ordinary launches of the combine paths: expert-side gather-reduce-push, owner-side sum.  Any grid size works.
// `reduce_ctas` reducer CTAs follow the args.forward_ctas forwarder CTAs in one grid.
cudaError_t launch_combine_push(const CombinePushArgs& args, int reduce_ctas, std::size_t smem, cudaStream_t stream);
cudaError_t launch_fused_reduce(const FusedReduceArgs& args, int ctas, cudaStream_t stream);
// True when the library was built with the per-role instrumentation (-DBEP_ENABLE_PROFILING=1).
bool role_profiling_enabled();

}  // namespace bep
