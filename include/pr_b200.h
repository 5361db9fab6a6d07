/* C ABI of libpr_b200.so: power retention (chunked forward/backward and
 * inference) as hand-written sm_100a kernels.
 *
 * Conventions for every entry point
 *   - returns PR_OK (0) or a negative PR_ERR_* code; pr_last_error() gives a
 *     thread-local message for the last failure on the calling thread;
 *   - never aborts, traps or allocates device memory: the caller passes every
 *     input, output and workspace as a raw device pointer (16-byte aligned);
 *   - work is enqueued on the given stream (a cudaStream_t passed as void*) of
 *     the given device ordinal; the call sets that device current itself, so it
 *     may be called from any thread (autograd's backward thread included);
 *   - `dtype` is PR_BF16 or PR_FP16 for Q/K/V-like tensors; gates, row sums and
 *     sum-of-keys tensors are always fp32.
 */
#ifndef PR_B200_H_
#define PR_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PR_ABI_VERSION 1

enum { PR_BF16 = 0, PR_FP16 = 1 };

enum {
  PR_OK = 0,
  PR_ERR_BAD_ARG = -1,     /* unsupported shape, null or misaligned pointer */
  PR_ERR_CUDA = -2,        /* a CUDA runtime/driver call failed */
  PR_ERR_TIMEOUT = -3,     /* a bounded device-side wait ran out */
  PR_ERR_UNSUPPORTED = -4  /* the device is not sm_100 */
};

int pr_abi_version(void);
const char* pr_last_error(void);

/* Reads (and clears) the status word that kernels of this library write when a
 * bounded device-side wait gives up.  Call after synchronising the stream.
 * *status is 0 when nothing failed. */
int pr_device_status(int device, int* status);

/* Self-test of the tensor-core building blocks on a 128 x N x K product:
 *   variant 0: A, B K-major in shared memory (manual swizzled stores)
 *   variant 1: A K-major, B MN-major in shared memory
 *   variant 2: A in tensor memory, B MN-major in shared memory
 *   variant 3: as 2, with B brought in by TMA
 *   variant 4: as 0, with A and B brought in by TMA
 * a: [128, k] row-major; b: [n, k] row-major for K-major variants, [k, n]
 * row-major for MN-major variants; out: [128, n] fp32.  k multiple of 64,
 * n in {64, 128, 256} (MN-major variants: n = 64). */
int pr_selftest_umma(int variant, int dtype, int n, int k, const void* a, const void* b, float* out,
                     int device, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* PR_B200_H_ */
