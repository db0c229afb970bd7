// Host entry point of the tcgen05 grouped expert GEMM (csrc/kernels/expert_gemm.cu).
#pragma once

#include <cuda_runtime.h>

namespace bep {

// out[rows of expert e, :] = A[rows of expert e, :] x W[e]^T, optionally with the SwiGLU epilogue
// (W[e] then holds 2n rows: gate rows first, up rows second).  A: [rows_capacity, k] bf16,
// W: [num_experts, (2)n, k] bf16, out: [rows_capacity, n] bf16; expert_offsets/[counts] are device
// int32 arrays as a dispatch produces them.  Returns nullptr on success, else a message.
const char* grouped_gemm_bf16(const void* a, const void* w, void* out, const int* expert_offsets, const int* expert_counts,
                              int* status, int rows_capacity, int num_experts, int n, int k, bool swiglu,
                              cudaStream_t stream);

}  // namespace bep
