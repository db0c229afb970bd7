// READY/ACK litmus over peer-visible memory (csrc/kernels/litmus.cu).
#pragma once

#include <cuda_runtime.h>

namespace bep {

// status: device int64 [4] (role 0/1) or [8] (role -1: producer then consumer):
//   {timed out, payload mismatches, rounds completed, elapsed ns}
// method 0: ordinary stores + st.release.sys; method 1: cp.async.bulk payload, completion wait, flag without a fence
const char* litmus_pingpong(void* mine, void* theirs, int role, int rounds, int words, long long* status,
                            unsigned long long timeout_ns, cudaStream_t stream, int method = 0);

}  // namespace bep
