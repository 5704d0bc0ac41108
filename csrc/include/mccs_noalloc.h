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
 * slice of the grid).
 *
 * Aliasing: any output may be exactly one of the inputs (out[r] == in[r'], for any r
 * and r': every element is read and then overwritten by the same thread). Buffers that
 * overlap without being identical (an output that starts inside an input) and two
 * outputs that share any part of their range, identical ones included, are rejected
 * with cudaErrorInvalidValue.
 *
 * Limits: 1 <= nranks <= MCCS_NOALLOC_MAX_RANKS; dtype float32, float16 or bfloat16
 * (mccsDataType_t numbering); sum only. Anything else is rejected with
 * cudaErrorInvalidValue before any work is queued. The scratch is
 * MCCS_NOALLOC_SCRATCH_BYTES per GPU that loads the library, held until exit.
 *
 * Rules for callers:
 *  - The first call on each device looks up the scratch array's device address, and the
 *    first launch of each kernel (one per element type) may make the CUDA runtime load
 *    code, which can allocate. Call mccsLocalAllReduceNoAllocPrepare() once per device
 *    before the window in which nothing may be allocated, and outside any stream
 *    capture; after it, mccsLocalAllReduceNoAlloc calls no allocating routine.
 *  - All calls on a device share the one scratch array, and each call first clears the
 *    part that must start at zero. Two calls that overlap on the GPU (different
 *    streams, no ordering between them) therefore race; order them.
 *  - The function queues work on `stream` and returns. A wait inside the kernel that
 *    runs out (10 s; it cannot in a correct launch, since all "ranks" are one grid) is
 *    recorded in the scratch array and reported by mccsLocalAllReduceNoAllocStatus,
 *    not by this function's return value, which only covers the launch.
 */
#ifndef MCCS_NOALLOC_H_
#define MCCS_NOALLOC_H_

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MCCS_NOALLOC_MAX_RANKS 8
#define MCCS_NOALLOC_SCRATCH_BYTES (8 * 5632)

/* Returns a cudaError_t value (0 = success). `in` and `out` are host arrays of `nranks`
 * device pointers; `stream` is a cudaStream_t. */
int mccsLocalAllReduceNoAlloc(const void* const* in, void* const* out, int nranks, size_t count, int dtype,
                              void* stream);

/* Everything that may allocate, done ahead of time for the current device: resolves the
 * scratch array's address and makes the runtime load the kernels of all three element
 * types. Returns a cudaError_t value. Not for use inside a stream capture. */
int mccsLocalAllReduceNoAllocPrepare(void);

/* What the kernels of the most recent call on the current device reported, per buffer
 * index: error[r] is 0, or 1 / 2 for a wait at the start / end of the kernel that ran
 * out, 4 for an abort, 5 for arguments the kernel refused; peer[r] names the buffer
 * index that was waited for. */
typedef struct {
  unsigned error[MCCS_NOALLOC_MAX_RANKS];
  unsigned peer[MCCS_NOALLOC_MAX_RANKS];
} mccsNoAllocStatus_t;

/* Waits for `stream` (the one the call was queued on), then copies the status words into
 * `*status` (plain host memory). Returns a cudaError_t value; allocates nothing. */
int mccsLocalAllReduceNoAllocStatus(mccsNoAllocStatus_t* status, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MCCS_NOALLOC_H_ */
