// Host entry point of the tcgen05 grouped expert GEMM (csrc/kernels/expert_gemm.cu).
#pragma once

#include <cuda_runtime.h>

#include "expert_gemm.cuh"

namespace bep {

// out[rows of expert e, :] = A[rows of expert e, :] x W[e]^T, optionally with the SwiGLU epilogue
// (W[e] then holds 2n rows: gate rows first, up rows second).  A: [rows_capacity, k], W: [num_experts, (2)n, k],
// both BF16 or both E4M3 (`fp8`; then a_scales [rows_capacity] and w_scales [num_experts, (2)n] are the
// per-row / per-output-channel FP32 scales applied in the epilogue); out: [rows_capacity, n] BF16;
// expert_offsets / expert_counts are device int32 arrays as a dispatch produces them.
// Returns nullptr on success, else a message.
const char* grouped_gemm(const void* a, const void* w, void* out, const float* a_scales, const float* w_scales,
                         const int* expert_offsets, const int* expert_counts, int* status, int rows_capacity,
                         int num_experts, int n, int k, bool swiglu, bool fp8, cudaStream_t stream);

// Plain BF16 GEMM (n a multiple of 256) whose epilogue, instead of writing an output matrix, multiplies each row
// by its routing weight and stores it into the token owner's landing slot (see gemm::ScatterTarget); the launch's
// last CTA publishes target.epoch to every rank.  Every launch on a device must use the same CTA count
// (grouped_gemm_ctas()) and consecutive epochs, because completion is detected with a monotonic counter.
const char* grouped_gemm_scatter(const void* a, const void* w, const int* expert_offsets, const int* expert_counts,
                                 int* status, int rows_capacity, int num_experts, int n, int k,
                                 const gemm::ScatterTarget& target, cudaStream_t stream);
int grouped_gemm_ctas();

}  // namespace bep
