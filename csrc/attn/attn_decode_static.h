/* Decode attention for callers that cannot allocate device memory.
 *
 * This entry point has no counterpart in the reference implementation.
 *
 * Some hosts of this library run where cudaMalloc is off limits: inside a process whose memory is
 * owned by another allocator with a fixed budget, in a real-time serving loop that forbids driver
 * allocation calls after start-up, or from a plug-in that may only pass pointers it was given.  The
 * regular entry point (ub_attn_decode) needs a scratch buffer for its split-KV partial results and
 * expects the caller to provide one.  ub_attn_decode_static_scratch runs the same kernels with that
 * scratch placed in a fixed array inside the library image instead, so the caller passes only its
 * inputs and outputs (args->scratch is ignored).
 *
 * Limits and rules:
 *  - The array holds UB_ATTN_STATIC_SCRATCH_FLOATS floats (16 MiB).  Every GPU that loads the library
 *    carries it until the process exits.  A call needs num_seqs * Hq * splits * (D + 2) floats; a call
 *    that needs more is rejected with UB_ERR_STATIC_SCRATCH_TOO_SMALL and launches nothing
 *    (ub_attn_decode_static_scratch_error() returns a sentence with both numbers).
 *  - The first call on each device looks up the array's device address (once per device, with that
 *    device current).  Make that first call before any stream capture begins on the device.
 *  - All calls share the one array and it keeps whatever the previous call left in it.  Nothing has
 *    to be cleared: each launch overwrites every partial slot it later reads.  For the same reason
 *    two calls that overlap in time on one GPU (different streams) race; run them one after the other.
 *  - No cudaMalloc, cudaFree or allocating library routine is called on any path of this function.
 */
#ifndef UNILLM_B200_ATTN_DECODE_STATIC_H_
#define UNILLM_B200_ATTN_DECODE_STATIC_H_
#include "../include/unillm_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

#define UB_ATTN_STATIC_SCRATCH_FLOATS (4u * 1024u * 1024u)
#define UB_ERR_STATIC_SCRATCH_TOO_SMALL (-20)
#define UB_ERR_STATIC_SCRATCH_SETUP (-21)

/* Same arguments and result as ub_attn_decode; args->scratch is ignored. */
int ub_attn_decode_static_scratch(const UbAttnArgs* args, void* stream);
/* Text of the last error reported by the function above on the calling thread ("" if none). */
const char* ub_attn_decode_static_scratch_error(void);

#ifdef __cplusplus
}
#endif
#endif
