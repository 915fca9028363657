/* Allocation-free entry points of libllmb200.
 *
 * This header has no counterpart in the reference project.
 *
 * Who needs it: some callers of this library are not allowed to create device memory at the
 * moment they call us.  Examples are code that runs inside another framework's memory pool and
 * must not call cudaMalloc behind its back, plugins that run after the process has handed all
 * free device memory to an arena, and service loops with a fixed memory budget where an
 * allocation (and the device synchronisation it can imply) is not acceptable.  The regular
 * bias-gradient entry point, llmb_dbias, takes a caller-provided scratch buffer; a caller that
 * cannot allocate has nothing to pass.  llmb_dbias_noalloc does the same reduction with its
 * scratch in a fixed array that lives inside the library image.
 */
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Upper limits of the built-in scratch: the partial sums occupy slabs*OC floats, where
 * slabs = llmb_dbias_slabs(rows) <= 128.  The array holds LLMB_DBIAS_NOALLOC_MAX_FLOATS floats
 * (4 MiB); every GPU that loads the library keeps that much memory reserved until the process
 * exits. */
#define LLMB_DBIAS_NOALLOC_MAX_FLOATS (1 << 20)

/* dbias[c] += sum over rows of dout[row, c], for c in [0, OC).
 *
 *   dbias  fp32 [OC], device memory, accumulated into (not overwritten)
 *   dout   [rows, OC] row-major, bf16 (dtype 1) or fp32 (dtype 0); OC a multiple of 8 (bf16) / 4 (fp32);
 *          the pointer must be 16-byte aligned (the kernels read rows with 16-byte loads; with those OC
 *          every row then is).  A misaligned pointer is refused with code 2.
 *   st     stream to launch on
 *
 * Returns 0 on success, 2 (bad argument) when llmb_dbias_slabs(rows)*OC exceeds
 * LLMB_DBIAS_NOALLOC_MAX_FLOATS or the shape is not supported, otherwise a cudaError_t value.
 * The call performs no cudaMalloc/cudaFree and calls no allocating library routine.
 *
 * First call on a device: the library looks up the device address of its scratch array once
 * per device (with that device current) and caches it.  Make that first call outside of any
 * stream capture, e.g. during start-up.
 *
 * Sharing: all calls on a device use the same scratch array.  Calls that may overlap on the
 * GPU (different streams without an ordering between them) race on it; issue them on one
 * stream or order them with events.  The array keeps the previous call's partial sums; the
 * kernels overwrite every element they later read, so nothing needs to be cleared.
 */
int llmb_dbias_noalloc(float* dbias, const void* dout, int rows, int OC, int dtype, cudaStream_t st);

#ifdef __cplusplus
}
#endif
