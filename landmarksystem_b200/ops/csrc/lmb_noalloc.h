/* Allocation-free entry point of liblmb200.
 *
 * This entry point has no counterpart in the reference system (LandMarkSystem); it exists for
 * callers of this library that are not allowed to allocate device memory at the point where they
 * need a prefix sum.
 *
 * Who that is: code that runs where cudaMalloc is off limits - a host thread inside a latency-critical
 * serving loop (cudaMalloc takes a driver lock and can stall every stream of the process), code that
 * runs after the framework has handed all device memory to a caching allocator it must not bypass,
 * and plug-ins loaded into a host application that owns the memory budget.  Such a caller passes
 * only its input and output buffers; the temporary storage the scan needs (per-tile partial sums)
 * lives in a fixed array inside the library instead of coming from an allocator.
 *
 *   int lmb_exclusive_scan_u32_noalloc(const uint32_t* in, uint32_t* out, long long n, cudaStream_t stream);
 *
 *   out[i] = in[0] + ... + in[i-1]  (mod 2^32) for 0 <= i < n; in and out are device pointers to n
 *   32-bit words each (out may alias in).  The work is enqueued on `stream`; the call does not
 *   synchronise.  Returns 0 on success, a positive cudaError_t value if the runtime reported one,
 *   or one of the negative codes below.  Results are identical to lmb_exclusive_scan_u32 with a
 *   caller-provided workspace.
 *
 * Limits and rules
 *   - n may not exceed LMB_NOALLOC_SCAN_MAX_ELEMS (16 Mi elements); larger requests are refused
 *     with LMB_NOALLOC_ERR_TOO_LARGE and nothing is launched.
 *   - The workspace is LMB_NOALLOC_SCAN_SCRATCH_BYTES (64 KiB) of device memory per GPU.  Every GPU
 *     whose context loads the library holds that much from load time until the process ends.
 *   - The first call on each device looks up the device address of the workspace (with that device
 *     current) and remembers it.  Make that first call outside of any stream capture.
 *   - All calls on one device share the one workspace, which still holds whatever the previous call
 *     left in it.  The scan overwrites every word before reading it, so no clearing is needed, but
 *     two calls whose kernels can overlap on the GPU (different streams without an ordering
 *     between them, or different host threads) race on it and give wrong sums.  Order them.
 *   - The call itself performs no cudaMalloc / cudaFree and calls no allocating library routine.
 */
#ifndef LMB_NOALLOC_H_
#define LMB_NOALLOC_H_

#include <cuda_runtime.h>
#include <stdint.h>

#define LMB_NOALLOC_SCAN_MAX_ELEMS (16LL * 1024 * 1024)
#define LMB_NOALLOC_SCAN_SCRATCH_BYTES (64 * 1024)

#define LMB_NOALLOC_ERR_ARGUMENT (-1000) /* null pointer or negative length */
#define LMB_NOALLOC_ERR_TOO_LARGE (-1001) /* n > LMB_NOALLOC_SCAN_MAX_ELEMS */
#define LMB_NOALLOC_ERR_DEVICE (-1002)    /* current device index outside the supported range */

#ifdef __cplusplus
extern "C" {
#endif

int lmb_exclusive_scan_u32_noalloc(const uint32_t* in, uint32_t* out, long long n, cudaStream_t stream);

#ifdef __cplusplus
}
#endif

#endif /* LMB_NOALLOC_H_ */
