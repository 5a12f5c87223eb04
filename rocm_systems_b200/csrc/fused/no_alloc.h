/*
 * An RMSNorm backward entry point for callers that are not allowed to allocate device memory.
 * It has no counterpart in the reference.
 *
 * Who needs it: code that runs where cudaMalloc is off limits — inside a latency-critical serving
 * loop whose memory budget was fixed at start-up, under a memory pool owned by another runtime
 * that forbids side allocations, or in a process that has already handed all device memory to a
 * framework allocator. The regular entry point (b200ops_rmsnorm_bwd) makes its caller provide an
 * fp32 accumulation buffer for the weight gradient; here that buffer is a fixed array that lives
 * inside the library image instead.
 *
 * What the call does: dx (bf16, [T, H]) and dw (bf16, [H]) of y = x * rstd * w, exactly as the
 * regular entry point followed by a cast of its fp32 weight gradient to bf16. The caller passes
 * every input and output; the only memory the call touches besides them is the library's own
 * scratch array.
 *
 * Limits and rules:
 *  - H must be a multiple of 8 and at most B200OPS_NOALLOC_MAX_H (8192). Larger rows are refused
 *    with B200OPS_NOALLOC_ERR_TOO_LARGE; nothing is launched.
 *  - The scratch is one array of B200OPS_NOALLOC_MAX_H floats (32 KiB) per GPU, resident from the
 *    moment the library is loaded on that GPU until the process exits.
 *  - The first call on each device looks up the device address of that array (with that device
 *    current). Make that first call outside of any stream capture. With lazy module loading the
 *    driver may also load this library's kernels, and take memory for them, during that first call:
 *    "allocates nothing" holds from the second call on a device onwards.
 *  - The address is kept for the life of the process. It does not survive cudaDeviceReset: a process
 *    that resets a device must not call this entry point on that device afterwards.
 *  - Every call uses the same array and leaves its last weight gradient in it; each call clears it
 *    first. Two calls that may overlap on one GPU (different streams, no ordering between them)
 *    race on it: order them, e.g. put them on one stream.
 *  - The call makes no cudaMalloc / cudaFree and uses no allocating library routine.
 */
#ifndef B200OPS_NO_ALLOC_H_
#define B200OPS_NO_ALLOC_H_

#include <cuda_runtime_api.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200OPS_NOALLOC_MAX_H 8192
#define B200OPS_NOALLOC_ERR_TOO_LARGE (-2)  /* H beyond B200OPS_NOALLOC_MAX_H (or not a multiple of 8) */
#define B200OPS_NOALLOC_ERR_SETUP (-3)      /* the scratch array's device address could not be obtained */

/* Returns 0 on success, one of the codes above, or a positive cudaError_t from a launch.
 * dy, x: [T, H] bf16; w: [H] bf16; rstd: [T] fp32 saved by the forward pass;
 * dx: [T, H] bf16 out; dwBf16: [H] bf16 out. */
int b200ops_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd, void* dx, void* dwBf16, long long T, int H,
                                cudaStream_t stream);

/* Text of the last refusal on this thread ("" when the last call went through). */
const char* b200ops_rmsnorm_bwd_noalloc_error(void);

#ifdef __cplusplus
}
#endif

#endif /* B200OPS_NO_ALLOC_H_ */
