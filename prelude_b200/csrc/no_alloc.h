/* Entry points of libprelude_b200 that allocate nothing.
 *
 * This part has no counterpart in the reference (Virtue-Research/prelude): it exists for callers of this
 * library that cannot obtain device memory at call time - a C or C++ host with a fixed memory plan and no
 * tensor library behind it, or code on a path where allocation is not allowed (while a stream is being
 * captured, inside a launch-path callback).
 */
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* out[r] = index of the largest of logits[r * row_stride .. + vocab), the smaller index on ties (the same
 * two-pass kernels as pb_argmax), for rows <= 256.  The scratch the two passes need is a 256 KB array built into
 * the library, one per GPU, held from library load until the process exits.
 *
 *  - No cudaMalloc, cudaFree or other allocating call is made.  Sizes beyond 256 rows are refused (return value
 *    non-zero, reason in pb_last_error()).
 *  - The first call on a device looks up the array's device address; make it before a stream capture begins.
 *  - Every call uses the same array, which keeps the previous call's contents.  Nothing needs to start at zero.
 *    Calls that overlap on the GPU (different streams or threads) race on it; calls on one stream do not.
 *  - The array that a call uses is the one of the device that is current when it is made.  logits, out and
 *    `stream` must belong to that device: make it current (cudaSetDevice) before the call.  Logits on another
 *    device are refused.
 *  - logits, out: device pointers; the launch goes to `stream`; nothing is synchronised.
 * Returns 0 on success. */
int pb_argmax_noalloc(const float* logits, long long row_stride, int rows, int vocab, int32_t* out,
                      cudaStream_t stream);

/* Message of the last failed call on this thread. */
const char* pb_last_error(void);

#ifdef __cplusplus
}
#endif
