/* Allocation-free local AllReduce.
 *
 * This entry point has no counterpart in the reference service: it exists for callers
 * that must not allocate device or pinned memory at the time they need a reduction —
 * code running while a memory pool is frozen or nearly exhausted, code inside a
 * section that forbids cudaMalloc (library callbacks, latency-critical loops that
 * cannot take the allocator's locks or an implicit device synchronisation), and
 * embedders that want a fixed memory footprint. Everything else in this library
 * gets its synchronisation scratch (signal pads, status blocks) from the daemon's
 * allocator; this function keeps that scratch in a file-scope device array instead.
 *
 * What it does: out[r][i] = sum over all r' of in[r'][i] for `nranks` buffers that all
 * live on the CURRENT device, written to every output buffer (the single-GPU form of
 * the two-shot AllReduce kernel: one cooperative launch in which each "rank" is a
 * slice of the grid). In place is allowed (out[r] == in[r]).
 *
 * Limits: 1 <= nranks <= MCCS_NOALLOC_MAX_RANKS; dtype float32, float16 or bfloat16
 * (mccsDataType_t numbering); sum only. Anything else is rejected with
 * cudaErrorInvalidValue before any work is queued. The scratch is
 * MCCS_NOALLOC_SCRATCH_BYTES per GPU that loads the library, held until exit.
 *
 * Rules for callers:
 *  - The first call on each device looks up the scratch array's device address. Make
 *    that first call outside any stream capture.
 *  - All calls on a device share the one scratch array, and each call first clears the
 *    part that must start at zero. Two calls that overlap on the GPU (different
 *    streams, no ordering between them) therefore race; order them.
 *  - The function queues work on `stream` and returns; it calls no allocating routine.
 */
#ifndef MCCS_NOALLOC_H_
#define MCCS_NOALLOC_H_

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MCCS_NOALLOC_MAX_RANKS 8
#define MCCS_NOALLOC_SCRATCH_BYTES (8 * 5120)

/* Returns a cudaError_t value (0 = success). `in` and `out` are host arrays of `nranks`
 * device pointers; `stream` is a cudaStream_t. */
int mccsLocalAllReduceNoAlloc(const void* const* in, void* const* out, int nranks, size_t count, int dtype,
                              void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MCCS_NOALLOC_H_ */
