/*
 * psdev_gemm_bf16_noalloc: the tcgen05 bf16 GEMM for callers that must not allocate.
 *
 * This entry point has no counterpart in the reference library (which has neither GPU code
 * nor any notion of device memory); it is an addition of this package.
 *
 * Who it is for.  psdev_gemm_bf16 obtains a small per-device scratch block (tile/CTA
 * counters and an error word) from cudaMalloc the first time it runs on a device.  Some
 * callers cannot afford that call: a serving process that has handed the whole device to a
 * framework's caching allocator, where a raw cudaMalloc may fail or fragment the pool; a
 * latency-critical thread that must never enter the driver's allocation path, which takes
 * process-wide locks and may synchronise the device; a host runtime that forbids any
 * allocation after start-up.  For them the scratch of this variant is a fixed array in the
 * library's own device data segment:
 *
 *   - size: 4352 bytes per GPU, held by every GPU that loads the library until the process
 *     exits, whether or not this function is ever called;
 *   - limit: the output may span at most 1023 column panels (N <= 1023 * 256 when N is a
 *     multiple of 256 or larger than 1024, N <= 1023 * 128 otherwise); larger N is rejected
 *     with PSDEV_ERR_TOO_LARGE and a message on stderr, and nothing is launched;
 *   - the function calls no cudaMalloc, cudaFree or other allocating routine; the caller
 *     supplies x, w, c and (optionally) the status word.
 *
 * First call on each device.  It looks up the device address of the scratch array (with that
 * device current) and raises the kernel's shared-memory limit.  Make that first call before
 * any stream capture begins on the device.
 *
 * Sharing.  Every call on a device uses the same array, which still holds what the previous
 * call left.  Each call therefore clears it, in stream order, before its kernel starts.  Two
 * calls whose kernels can overlap on one GPU (different streams, or different host threads
 * without ordering between them) race on the array and give undefined results; issue them
 * on one stream or order them with events.  psdev_gemm_bf16 uses a different scratch block, so
 * its calls may overlap calls of this function.
 *
 * Arguments as for psdev_gemm_bf16 (c[M,N] = x[M,K] * w[N,K]^T, row-major bf16, 16-byte
 * aligned, N and K multiples of 8).  `status_dev`, if not NULL, is a device pointer to an
 * int32 that receives, in stream order after the kernel, 0 or the negative psdev error the
 * kernel recorded (for instance PSDEV_ERR_TIMEOUT_PIPE).  It is the only way to learn of an
 * error inside the kernel: the next call clears the array, error word included, and
 * psdev_gemm_status reads the other entry points' scratch block, not this one.  A caller that
 * passes NULL gives that information up.
 * Returns 0, a negative psdev error, or a positive cudaError_t.
 */
#ifndef PS_KERNELS_PULL_GEMM_NOALLOC_H_
#define PS_KERNELS_PULL_GEMM_NOALLOC_H_
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PSDEV_ERR_TOO_LARGE (-7)
#define PSDEV_NOALLOC_SCRATCH_BYTES 4352

int psdev_gemm_bf16_noalloc(const void* x, const void* w, void* c, int64_t M, int64_t N,
                            int64_t K, int num_ctas, uint64_t timeout_ns, int32_t* status_dev,
                            void* stream);

#ifdef __cplusplus
}
#endif
#endif /* PS_KERNELS_PULL_GEMM_NOALLOC_H_ */
