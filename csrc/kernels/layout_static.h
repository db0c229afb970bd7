/* Routing layout without any allocation.
 *
 * This entry point has no counterpart in the reference project.
 *
 * Who it is for: code that may not call cudaMalloc at the point where it needs a routing plan -- an
 * inference server whose memory is handed out once at start-up by its own arena, a plugin running
 * inside another framework's allocator, or a latency-critical section where the implicit
 * device-wide synchronisation of cudaMalloc/cudaFree is not acceptable.  Every other entry point of
 * this library keeps its cross-CTA scratch (per-channel histograms and a barrier counter) in memory
 * that the runtime allocates when a buffer is built; this one keeps it in a fixed array inside the
 * loaded library instead, so the caller passes nothing but its inputs and outputs.
 *
 * What it computes: exactly the plan that the dispatch kernel's layout phase produces for one rank's
 * topk_idx (the four arrays a dispatch result exposes through its layout object):
 *   plan_mask[T]          bit d set  <=> token goes to rank d
 *   plan_slot[T][P]       channel-relative row index of the token at rank d, -1 if not sent there
 *   plan_expert_ord[T][K] stable ordinal of the token among this rank's tokens of that expert, -1 for
 *                         unused slots
 *   plan_counts[P+E+C*P]  tokens per destination rank, routes per expert, tokens per (channel, rank)
 *
 * Limits (the scratch array is sized for them; larger requests are rejected, nothing is truncated):
 *   num_channels <= 64, num_experts <= 1024, num_ranks <= 16, num_topk <= 32.
 *   The array is 266,496 bytes; every GPU that loads the library holds it until the process exits.
 *
 * Rules for callers:
 *   - The first call on a device looks up the array's device address (cudaGetSymbolAddress) and the
 *     kernel's occupancy; make that first call outside any stream capture.
 *   - All calls on one device share the one scratch array.  Two calls whose kernels may overlap on
 *     the GPU (different streams without an ordering between them) race on it; order them.
 *   - `status` is an output: 4 ints in device memory, zero on success; status[0] = 2 reports an
 *     invalid route (expert id out of range or repeated within a token; status[1] = token,
 *     status[2] = slot), status[0] = 21 a barrier that did not complete within 2 s.
 *   - When status[0] != 0 the four plan arrays hold unspecified values (the dispatch kernel never
 *     uses a plan either once it has seen an invalid route): read `status` before the plan.
 *   - num_tokens = 0 is a valid request (the counts come out zero; the per-token arrays may then be
 *     null), and so is num_channels > num_tokens (the surplus channels own no token).
 *   - All pointers are device pointers on the current device; topk_idx is int64 [T][K], contiguous.
 *
 * Return value: 0 on success (the work is enqueued on `stream`), a positive cudaError_t value if a
 * CUDA call failed, or one of the negative codes below if the request was refused.
 */
#pragma once

#include <stdint.h>

#include <cuda_runtime_api.h>

#ifdef __cplusplus
extern "C" {
#endif

#define BEP_STATIC_MAX_CHANNELS 64
#define BEP_STATIC_MAX_EXPERTS 1024
#define BEP_STATIC_MAX_RANKS 16
#define BEP_STATIC_MAX_TOPK 32

#define BEP_STATIC_ERR_TOO_LARGE (-1)   /* a dimension exceeds the limits above            */
#define BEP_STATIC_ERR_ARGUMENT (-2)    /* null pointer, negative size, experts % ranks    */
#define BEP_STATIC_ERR_RESIDENCY (-3)   /* num_channels CTAs cannot be co-resident here    */

__attribute__((visibility("default"))) int bep_route_layout_static(
    const int64_t* topk_idx, int num_tokens, int num_topk, int num_experts, int num_ranks, int num_channels,
    uint32_t* plan_mask, int* plan_slot, int* plan_expert_ord, int* plan_counts, int* status, cudaStream_t stream);

/* Size in bytes of the library-resident scratch array (for accounting). */
__attribute__((visibility("default"))) unsigned long long bep_route_layout_static_scratch_bytes(void);

#ifdef __cplusplus
}
#endif
