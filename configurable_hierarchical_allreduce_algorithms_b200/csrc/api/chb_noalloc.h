/* Allocation-free one-shot allreduce for ranks that share one GPU.
 *
 * This entry point has no counterpart in the reference (which only ever uses
 * malloc'ed host buffers); it exists for callers of this library that are not
 * allowed to allocate device memory at the point where they need a
 * collective: code that runs while a memory pool is frozen or nearly full,
 * plugins that are handed their buffers by a host framework and must not touch
 * the allocator, and latency-critical loops in which a cudaMalloc (which
 * synchronises the device) would stall everything else.  Such callers cannot
 * create a communicator, because a communicator owns a symmetric heap, control
 * blocks and program tables that are all allocated.
 *
 * chb_allreduce_oneshot_noalloc() reduces P equally long vectors that live on
 * the current GPU (the "emulated world" of this library: P ranks on one
 * device) with the flagged-line one-shot algorithm and writes the full result
 * to each of the P outputs.  Its only working memory is a fixed array that is
 * part of the library image:
 *
 *   - capacity: at most CHB_NOALLOC_MAX_RANKS ranks and CHB_NOALLOC_MAX_BYTES
 *     payload bytes per rank; larger requests are refused with CHB_ERR_COUNT
 *     and a message, nothing is launched;
 *   - cost: every GPU that loads the library holds the array
 *     (about 1.1 MiB) until the process exits;
 *   - the array is shared by all calls and keeps the previous call's contents.
 *     Each call therefore first clears, on `stream`, the control words and the
 *     inbox lines it is going to use.  Two calls whose kernels can overlap on
 *     the GPU (different streams without ordering between them, or two host
 *     threads) race on that array and give wrong results: order them;
 *   - the first call on a device looks up the array's device address
 *     (cudaGetSymbolAddress, with that device current) and remembers it.  Make
 *     that first call outside of any stream capture.  The per-device table of
 *     remembered addresses is written without a lock: two host threads that
 *     make the first call on one device at the same time both store the same
 *     value, which is harmless;
 *   - no cudaMalloc / cudaFree / allocating library routine is called, on the
 *     first call or later.
 *
 * in / out: arrays of P device pointers (8-byte aligned, `count` elements
 * each, on the current device).  dtype / op: the CHB_* enums of chb.h.
 * `scale` multiplies the reduced values once.  Waits inside the kernel are
 * bounded (about two seconds); if one expires the outputs are undefined and
 * the next call to chb_noalloc_status() reports it.
 * Returns CHB_SUCCESS or a CHB_ERR_* code; on error a message is copied to
 * err (if not NULL).
 */
#ifndef CHB_NOALLOC_H_
#define CHB_NOALLOC_H_
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define CHB_NOALLOC_MAX_RANKS 8
#define CHB_NOALLOC_MAX_BYTES 8192

int chb_allreduce_oneshot_noalloc(int P, int dtype, int op, const void* const* in, void* const* out,
                                  int64_t count, float scale, cudaStream_t stream, char* err, int errlen);

/* Synchronises `stream` and returns CHB_SUCCESS, or CHB_ERR_TIMEOUT if a wait
 * of the last call on the current device expired.  Allocates nothing. */
int chb_noalloc_status(cudaStream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* CHB_NOALLOC_H_ */
