/* fluxb_moe_index_build_static: the MoE routing-index build for callers that must not
 * allocate device memory. This entry point has no counterpart in the reference library.
 *
 * Who needs it: a host program that gave all device memory to its own arena at start-up (an
 * inference server with a pre-sized pool has nothing left for a side allocation), or one whose
 * request loop may not call cudaMalloc at all because that call synchronises the whole device
 * and stalls every stream. fluxb_moe_index_build asks such a caller for a scratch buffer of
 * fluxb_moe_index_scratch_elems(n, E) int32; this variant needs none. Inputs and outputs are
 * still the caller's.
 *
 * The scratch is a fixed array of FLUXB_MOE_INDEX_STATIC_ELEMS int32 (1 MiB) that lives in the
 * library image: every GPU that loads libfluxb holds that 1 MiB until the process exits.
 * A problem fits when ceil(n / 4096) * E <= FLUXB_MOE_INDEX_STATIC_ELEMS (for E = 64 that is
 * about 16.7 million routed entries); larger problems are refused with error code 1 and a
 * message, nothing is launched.
 *
 * The first call on a device looks up the device address of the array, once, with that device
 * current. Make that first call before any stream capture begins; it may come from any host
 * thread, also from several at once (the cached address is an atomic). No call of this entry point
 * uses cudaMalloc, cudaFree or any allocating library routine.
 *
 * All calls on a device share the one array, and it keeps whatever the last call left in it.
 * Nothing in it has to start at zero: each call rewrites every word it later reads. Two calls
 * whose kernels overlap on the GPU (different streams, no dependency between them) race on the
 * array and give wrong indices; order them on one stream or with events.
 *
 * Arguments and results are those of fluxb_moe_index_build without `scratch`. */
#ifndef FLUXB_MOE_INDEX_STATIC_H_
#define FLUXB_MOE_INDEX_STATIC_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FLUXB_MOE_INDEX_STATIC_ELEMS (256 * 1024)

int fluxb_moe_index_build_static(const int32_t* experts, int64_t n, int E, int topk,
                                 int32_t* splits, int32_t* offsets, int32_t* scatter_index,
                                 int32_t* gather_index, int32_t* topk_index, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FLUXB_MOE_INDEX_STATIC_H_ */
