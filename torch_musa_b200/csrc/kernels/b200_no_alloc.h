/* Allocation-free entry point of libb200_kernels.so.
 *
 * This entry point has no counterpart in the reference; it exists for callers of this library that are
 * not allowed to allocate device memory at the moment they need the result: code running inside a
 * region where the driver allocator must not be entered (a real-time control loop, a signal-safe or
 * out-of-memory diagnostic path, a host application that has handed all device memory to its own
 * arena and exposes no allocator to plug-ins).  Such a caller cannot provide the scratch buffer that
 * b200_multi_tensor_l2norm() needs, and this library must not call cudaMalloc on its behalf.
 *
 * b200_multi_tensor_l2norm_static() computes the same result as b200_multi_tensor_l2norm() -- the L2
 * norm of every tensor of a list and the norm over the whole list -- but keeps its partial sums in a
 * fixed array that is part of the library image on every GPU that loads it.
 *
 *   Limit     at most B200_L2NORM_STATIC_MAX_TENSORS (1024) tensors per call; more is refused with
 *             cudaErrorInvalidValue and nothing is launched.  The array is 1024 * 321 + 8 floats
 *             (about 1.3 MB) and stays resident on each device until the process exits.
 *   Set-up    the first call on a device looks up the array's device address (with that device
 *             current) and caches it; make that first call before starting any stream capture.  The
 *             first call on a device may come from any thread: concurrent first calls all store the
 *             same address into the cache, so no lock is taken.
 *   Sharing   every call on a device uses the same array and leaves its partial sums behind.  Each
 *             call overwrites every slot it later reads, so nothing has to be cleared between calls,
 *             but two calls that overlap on the GPU (different streams, no ordering) race on the
 *             array and produce garbage: serialise them.
 *   No allocation: neither cudaMalloc/cudaFree nor any allocating library routine is called.
 *
 * Inputs and outputs are the caller's: `tensors` / `numels` are host arrays of n device pointers and
 * element counts, `out_total` (1 float) and `out_per_tensor` (n floats, may be NULL) are device
 * pointers.  Returns a cudaError_t value as int.
 */
#pragma once

#include "b200_kernels.h"

#ifdef __cplusplus
extern "C" {
#endif

#define B200_L2NORM_STATIC_MAX_TENSORS 1024

B200_API int b200_multi_tensor_l2norm_static(int n_tensors, int dtype, void* const* tensors, const int64_t* numels,
                                             float* out_total, float* out_per_tensor, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
